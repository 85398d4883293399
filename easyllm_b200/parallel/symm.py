"""Symmetric-memory workspace of the fused tensor-parallel kernels.

Every rank of the TP group owns, at the same offsets of one symmetric allocation (CUDA VMM
memory mapped on all peers through ``torch.distributed._symmetric_memory``):

  gathered [2][T, hidden] bf16  all-gather→GEMM: rank s copies its sequence shard into rows
                              ``[s·T/tp, (s+1)·T/tp)`` of every rank's buffer; two buffers alternate by
                              call so a following kernel (wgrad) can still read the previous gather
  staging  [T, hidden] bf16   GEMM→reduce-scatter: this rank's partial product, read by the owners
  flags / done words          epoch counters written by peers (one set per kernel kind)

The kernels (``csrc/gemm.cu``: ``ell_gemm_ag`` / ``ell_gemm_rs``) receive the peers' base
pointers and move data with plain NVLink loads/stores issued from inside the GEMM kernel;
only local memory is ever read by TMA.  ``install()`` registers them with ``tp_linear`` so
Column/RowParallelLinear use them for CUDA bf16 inputs; the NCCL composition remains the
fallback (shapes that do not tile, CPU) and the A/B baseline.

Replaces the per-linear ``_all_gather_base`` / ``_reduce_scatter_base`` calls of the
reference (llm/models/mg_models/base_modules/layers/column_parallel_linear.py:29-38,87-95,
row_parallel_linear.py:116-117).
"""
from __future__ import annotations

import os
from ctypes import c_int, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..utils.log import default_logger as logger
from .grid import get_grid

_MAX_FLAGS = 8192        # flag words per source rank
_N_COMM_AG = 8
_N_COMM_RS = 8


class FusedTPWorkspace:
    def __init__(self, max_tokens, hidden, group=None, n_comm_ag=_N_COMM_AG, n_comm_rs=_N_COMM_RS):
        import torch.distributed._symmetric_memory as symm_mem
        g = get_grid()
        self.group = group if group is not None else g.tp_group
        self.tp, self.rank = g.tp, g.tp_rank
        self.max_tokens, self.hidden = max_tokens, hidden
        self.n_comm_ag = int(os.environ.get("ELL_NCOMM_AG", n_comm_ag))
        self.n_comm_rs = int(os.environ.get("ELL_NCOMM_RS", n_comm_rs))
        if "ELL_RS_ORDER" in os.environ:              # tuning: "interleaved" (default) or "ring"
            from ..ops import cuda as cu
            cu.lib().ell_gemm_set_rs_order(c_int(1 if os.environ["ELL_RS_ORDER"] == "ring" else 0))
        dev = torch.device("cuda", torch.cuda.current_device())
        data_elems = max_tokens * hidden
        flag_words = 2 * (self.tp * _MAX_FLAGS + 64)             # AG set + RS set (flags + done)
        nbytes = 3 * data_elems * 2 + flag_words * 4            # gathered x2 (alternating by epoch) + staging
        name = self.group.group_name
        try:
            symm_mem.enable_symm_mem_for_group(name)
        except Exception:
            pass
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=name)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        base = [int(p) for p in self.hdl.buffer_ptrs]
        off_stage = 2 * data_elems * 2
        off_flags = 3 * data_elems * 2
        set_bytes = (self.tp * _MAX_FLAGS + 64) * 4
        # two gathered buffers used alternately: a later kernel on this stream (the wgrad GEMM) may still read
        # epoch e's gathered operand while fast peers already push epoch e+1
        self.gathered_ptrs = [base, [b + data_elems * 2 for b in base]]
        self._gathered_off = [0, data_elems * 2]
        self.stage_ptrs = [b + off_stage for b in base]
        self.ag_flags = [b + off_flags for b in base]
        self.ag_done = [b + off_flags + self.tp * _MAX_FLAGS * 4 for b in base]
        self.rs_flags = [b + off_flags + set_bytes for b in base]
        self.rs_done = [b + off_flags + set_bytes + self.tp * _MAX_FLAGS * 4 for b in base]
        self.counters = torch.zeros(4, dtype=torch.int32, device=dev)   # [ag done-count, -, rs done-count, rs queue]
        self.epoch_ag = 0
        self.epoch_rs = 0
        self.rs_queue = 0
        self._arr = lambda ptrs: (c_void_p * len(ptrs))(*ptrs)
        logger.info(f"fused TP workspace: {nbytes / 2**20:.0f} MiB symmetric memory over {self.tp} ranks")

    # ------------------------------------------------------------------------------------------
    def _ok(self, rows_per_rank, width):
        return (rows_per_rank % 128 == 0 and rows_per_rank * self.tp <= self.max_tokens and width <= self.hidden
                and width % 8 == 0)

    def ag_gemm(self, x_local, w, bias=None, b_mn=False):
        """``gather(x_local) · wᵀ (+bias)`` (``w [N, K]``), or with ``b_mn`` ``gather(x_local) · w`` (``w [K, N]``);
        returns ``[T, N]`` or None when the shape is unsupported."""
        from ..ops import cuda as cu
        rows, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if not self._ok(rows, K) or rows // 128 > _MAX_FLAGS or N % 8 or (b_mn and bias is not None):
            return None
        x_local = x_local.contiguous()
        out = torch.empty(rows * self.tp, N, dtype=torch.bfloat16, device=x_local.device)
        self.epoch_ag += 1
        rc = cu.lib().ell_gemm_ag(cu._p(x_local), cu._p(w), cu._p(out), cu._p(bias), c_int(rows), c_int(N), c_int(K),
                                  c_int(1 if b_mn else 0), c_int(self.rank), c_int(self.tp), c_uint(self.epoch_ag), c_int(self.n_comm_ag),
                                  self._arr(self.gathered_ptrs[self.epoch_ag & 1]), self._arr(self.ag_flags), self._arr(self.ag_done),
                                  c_void_p(self.counters.data_ptr()), c_int(_MAX_FLAGS),
                                  cu._p(cu.err_flag(x_local.device)), cu._stream())
        cu._check(rc, "gemm_ag")
        self._last_ag = (x_local, rows, K, self._gathered_off[self.epoch_ag & 1])
        return out

    def gathered(self):
        """The all-gathered operand ``[T, K]`` of the last ``ag_gemm`` (a view into the workspace, valid until the
        next fused call).  Peers' shards were pushed by the kernel; the local shard is copied in here."""
        x_local, rows, K, off = self._last_ag
        full = self.buf[off: off + rows * self.tp * K * 2].view(torch.bfloat16).view(rows * self.tp, K)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_local)
        return full

    def gemm_rs(self, x, w, b_mn=False):
        """reduce-scatter over TP of ``x · op(w)``; returns this rank's ``[T/tp, N]`` rows or None."""
        from ..ops import cuda as cu
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if M % self.tp:
            return None
        rows = M // self.tp
        bn = 256 if N >= 256 else 128
        tiles_n = (N + bn - 1) // bn
        if not self._ok(rows, N) or N % bn or (rows // 128) * tiles_n > _MAX_FLAGS or K % 8:
            return None
        x = x.contiguous()
        y = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
        self.epoch_rs += 1
        rc = cu.lib().ell_gemm_rs(cu._p(x), cu._p(w), cu._p(y), c_int(rows), c_int(N), c_int(K), c_int(1 if b_mn else 0),
                                  c_int(self.rank), c_int(self.tp), c_uint(self.epoch_rs), c_int(self.n_comm_rs),
                                  self._arr(self.stage_ptrs), self._arr(self.rs_flags), self._arr(self.rs_done),
                                  c_void_p(self.counters.data_ptr() + 8), c_int(_MAX_FLAGS),
                                  c_uint(self.rs_queue & 0xFFFFFFFF), cu._p(cu.err_flag(x.device)), cu._stream())
        cu._check(rc, "gemm_rs")
        self.rs_queue += cu.lib().ell_gemm_rs_queue_advance(c_int(rows), c_int(N))
        return y


_WS = None


def install(max_tokens, hidden):
    """Create the workspace for this TP group and route the TP linears through the fused kernels."""
    global _WS
    from . import tp_linear
    g = get_grid()
    if g.tp == 1 or not torch.cuda.is_available():
        return None
    _WS = FusedTPWorkspace(max_tokens, hidden)

    def ag(x, w, bias, b_mn=False, want_gathered=False):
        y = _WS.ag_gemm(x, w, bias, b_mn)
        if y is None:
            return None
        return (y, _WS.gathered() if want_gathered else None)

    def rs(x, w, b_mn=False):
        return _WS.gemm_rs(x, w, b_mn)

    tp_linear.set_fused_impl(ag, rs)
    return _WS


def uninstall():
    global _WS
    from . import tp_linear
    tp_linear.set_fused_impl(None, None)
    _WS = None


def workspace():
    return _WS
