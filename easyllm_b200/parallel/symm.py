"""Symmetric-memory workspace of the fused tensor-parallel kernels.

Every rank of the TP group owns, at the same offsets of one symmetric allocation (CUDA VMM
memory mapped on all peers through ``torch.distributed._symmetric_memory``):

  gathered [2][T, hidden] bf16  all-gather→GEMM: rank s copies its sequence shard into rows
                              ``[s·T/tp, (s+1)·T/tp)`` of every rank's buffer; two buffers alternate by
                              call so a following kernel can still read the previous gather
  staging  [T, hidden] bf16   GEMM→reduce-scatter on CTA pairs: rows ``[s·T/tp, (s+1)·T/tp)`` receive rank s's
                              partial sums of the tiles THIS rank owns (written by s through its peer pointer,
                              added in the owner's GEMM epilogue); GEMM→all-reduce and the single-CTA
                              reduce-scatter: this rank's partial product (and, for the all-reduce, the
                              reduced tiles it owns), read by the peers
  flags / done words          epoch counters written by peers (one set per kernel kind)
  ce      [2][tp][T, 3] fp32  cross-entropy statistics pushed by every rank (two buffers alternate by call)

The kernels (``csrc/gemm_pair.cu`` on CTA pairs, ``csrc/gemm.cu`` for shapes whose row shards are not a
multiple of 256) receive the peers' base pointers and move data with plain NVLink loads/stores issued from
inside the GEMM kernel; only local memory is ever read by TMA.  ``install()`` registers them with
``tp_linear`` so Column/RowParallelLinear use them for CUDA bf16 inputs; the NCCL composition remains for
shapes that do not tile (logged once, an error under strict mode) and as the A/B baseline.

Replaces the per-linear ``_all_gather_base`` / ``_reduce_scatter_base`` / ``all_reduce`` calls of the
reference (llm/models/mg_models/base_modules/layers/column_parallel_linear.py:29-38,53-61,87-95,
row_parallel_linear.py:116-119, llm/models/mg_models/llama/lm_head.py:53-57,
base_modules/functions/cross_entropy.py:35-37,67-69,78-80).
"""
from __future__ import annotations

from ctypes import c_int, c_longlong, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..utils.log import default_logger as logger
from .grid import get_grid

_MAX_FLAGS = 8192        # flag words per source rank
_N_COMM_AG = 8           # communication CTAs of a gather launch (even: whole two-CTA clusters)


def _u32(v):
    return c_uint(v & 0xFFFFFFFF)


class FusedTPWorkspace:
    def __init__(self, max_tokens, hidden, group=None, n_comm_ag=_N_COMM_AG, n_comm_rs=None):
        import torch.distributed._symmetric_memory as symm_mem
        g = get_grid()
        self.group = group if group is not None else g.tp_group
        self.tp, self.rank = g.tp, g.tp_rank
        self.max_tokens, self.hidden = max_tokens, hidden
        self.n_comm_ag = int(n_comm_ag)
        self.n_comm_rs_fixed = None if n_comm_rs is None else int(n_comm_rs)   # None: chosen per launch from K
        dev = torch.device("cuda", torch.cuda.current_device())
        data_elems = max_tokens * hidden
        set_words = self.tp * _MAX_FLAGS + 64                     # flags of one kind + its done words
        flag_words = 4 * set_words                               # gather, reduce partials, reduced tiles, ce
        ce_bytes = 2 * self.tp * max_tokens * 3 * 4
        nbytes = 3 * data_elems * 2 + flag_words * 4 + ce_bytes  # gathered x2 (alternating by epoch) + staging
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
        set_bytes = set_words * 4
        # two gathered buffers used alternately: a later kernel on this stream may still read epoch e's gathered
        # operand while fast peers already push epoch e+1
        self.gathered_ptrs = [base, [b + data_elems * 2 for b in base]]
        self._gathered_off = [0, data_elems * 2]
        self.stage_ptrs = [b + off_stage for b in base]
        self.ag_flags = [b + off_flags for b in base]
        self.ag_done = [b + off_flags + self.tp * _MAX_FLAGS * 4 for b in base]
        self.rs_flags = [b + off_flags + set_bytes for b in base]
        self.rs_done = [b + off_flags + set_bytes + self.tp * _MAX_FLAGS * 4 for b in base]
        self.red_flags = [b + off_flags + 2 * set_bytes for b in base]
        self.ce_flags = [b + off_flags + 3 * set_bytes for b in base]
        self.ce_bufs = [b + off_flags + 4 * set_bytes for b in base]
        self.counters = torch.zeros(4, dtype=torch.int32, device=dev)   # [ag cta count, -, rs cta count, rs queue]
        self.epoch_ag = self.epoch_rs = self.epoch_ce = 0
        self._pushed = None                                     # (ptr, rows, K, epoch) of a push awaiting its consumer
        self.ag_count = self.rs_count = self.rs_queue = 0       # host copies of the device counters
        self._arr = lambda ptrs: (c_void_p * len(ptrs))(*ptrs)
        from ..ops import cuda as cu
        lib = cu.lib()
        from ctypes import c_ulonglong
        lib.ell_gemm_set_fused_buffer_bytes(c_ulonglong(data_elems * 2))   # the kernels check tile offsets against it
        self.grid_single = lib.ell_gemm_fused_grid()
        self.grid_pair = lib.ell_gemm_pair_fused_grid()
        self.use_pair = cu.gemm_pair_enabled() and self.grid_pair > 0
        logger.info(f"fused TP workspace: {nbytes / 2**20:.0f} MiB symmetric memory over {self.tp} ranks; "
                    f"{'CTA-pair' if self.use_pair else 'single-CTA'} kernels")

    # ------------------------------------------------------------------------------------------
    def _refuse(self, op, t, why):
        from .. import ops
        ops.note_fallback(op, t, why)
        return None

    def _ok(self, op, t, rows_per_rank, width):
        why = None
        if rows_per_rank % 128:
            why = f"{rows_per_rank} rows per rank is not a multiple of 128"
        elif rows_per_rank * self.tp > self.max_tokens or width > self.hidden:
            why = f"{rows_per_rank * self.tp} x {width} exceeds the workspace ({self.max_tokens} x {self.hidden})"
        elif width % 8:
            why = f"width {width} is not a multiple of 8"
        if why is not None:
            self._refuse(op, t, why)
        return why is None

    def _reduce_ctas(self, K):
        """Dedicated reduce CTAs of a launch with a staged reduction (GEMM→all-reduce, single-CTA reduce-scatter; the
        CTA-pair reduce-scatter sums in its epilogue and has none).  The reduction moves a fixed number of bytes per
        output tile while the GEMM time per tile grows with K: a short reduction dimension needs more CTAs summing
        tiles during the main loop, or the whole reduction is left for the tail (about 30000 / K of them keep
        pace; even, because the CTA-pair kernel hands out whole clusters)."""
        if self.n_comm_rs_fixed is not None:
            return self.n_comm_rs_fixed
        n = int(round(30000.0 / max(K, 1)))
        return max(4, min(32, n + (n & 1)))

    def _pair(self, rows_per_rank, N):
        return self.use_pair and rows_per_rank % 256 == 0 and N >= 256

    def _ag_args(self):
        self.epoch_ag += 1
        return (self._arr(self.gathered_ptrs[self.epoch_ag & 1]), self._arr(self.ag_flags), self._arr(self.ag_done),
                c_void_p(self.counters.data_ptr()), _u32(self.ag_count), c_int(_MAX_FLAGS))

    def ag_gemm(self, x_local, w, bias=None, b_mn=False):
        """``gather(x_local) · wᵀ (+bias)`` (``w [N, K]``), or with ``b_mn`` ``gather(x_local) · w`` (``w [K, N]``);
        returns ``[T, N]`` or None when the shape is unsupported."""
        from ..ops import cuda as cu
        rows, K = x_local.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if not self._ok("ag_gemm", x_local, rows, K):
            return None
        if rows // 128 > _MAX_FLAGS or N % 8 or (b_mn and bias is not None):
            return self._refuse("ag_gemm", x_local, f"N = {N} / bias with a transposed weight")
        x_local = x_local.contiguous()
        out = torch.empty(rows * self.tp, N, dtype=torch.bfloat16, device=x_local.device)
        lib = cu.lib()
        pair = self._pair(rows, N)
        head = (cu._p(x_local), cu._p(w), cu._p(out), cu._p(bias), c_int(rows), c_int(N), c_int(K),
                c_int(1 if b_mn else 0), c_int(self.rank), c_int(self.tp))
        ptrs = self._ag_args()
        tail = (cu._p(cu.err_flag(x_local.device)), cu._stream())
        if pair:
            rc = lib.ell_gemm_ag_pair(*head, _u32(self.epoch_ag), c_int(self.n_comm_ag), *ptrs, c_void_p(0), c_void_p(0),
                                      c_longlong(0), c_int(0), *tail)
            self.ag_count += self.grid_pair - self.n_comm_ag
        else:
            rc = lib.ell_gemm_ag(*head, _u32(self.epoch_ag), c_int(self.n_comm_ag), *ptrs, *tail)
            self.ag_count += self.grid_single - self.n_comm_ag
        cu._check(rc, "gemm_ag")
        self._last_ag = (x_local, rows, K, self._gathered_off[self.epoch_ag & 1])
        return out

    def ag_gemm_ce(self, x_local, w, target, vocab_start, valid_cols):
        """LM head behind the sequence-parallel gather with the cross-entropy statistics in the epilogue:
        returns ``(logits [T, V] bf16, parts [T, 3] fp32)`` or None (see ``ops.cuda.gemm_ce``)."""
        from ..ops import cuda as cu
        rows, K = x_local.shape
        V = w.shape[0]
        if not self._ok("ag_gemm_ce", x_local, rows, K):
            return None
        if not self._pair(rows, V) or V % 8:
            return self._refuse("ag_gemm_ce", x_local, "needs the CTA-pair kernel (rows per rank a multiple of 256)")
        x_local = x_local.contiguous()
        T = rows * self.tp
        logits = torch.empty(T, V, dtype=torch.bfloat16, device=x_local.device)
        lib = cu.lib()
        slots = lib.ell_gemm_ce_slots_pair(c_int(V))
        part = cu.scratch(slots * 3 * T, tag="gemm_ce_part")
        parts = torch.empty(T, 3, dtype=torch.float32, device=x_local.device)
        tgt = (target if target.dtype == torch.int64 else target.to(torch.int64)).contiguous()
        ptrs = self._ag_args()
        rc = lib.ell_gemm_ag_pair(cu._p(x_local), cu._p(w), cu._p(logits), c_void_p(0), c_int(rows), c_int(V), c_int(K),
                                  c_int(0), c_int(self.rank), c_int(self.tp), _u32(self.epoch_ag), c_int(self.n_comm_ag),
                                  *ptrs, cu._p(tgt), cu._p(part), c_longlong(vocab_start), c_int(valid_cols),
                                  cu._p(cu.err_flag(x_local.device)), cu._stream())
        self.ag_count += self.grid_pair - self.n_comm_ag
        cu._check(rc, "gemm_ag_ce")
        cu._check(lib.ell_ce_combine(cu._p(part), cu._p(parts), c_int(slots), c_int(T), cu._stream()), "ce_combine")
        self._last_ag = (x_local, rows, K, self._gathered_off[self.epoch_ag & 1])
        return logits, parts

    def agk_accepts(self, dy, x_local, dw32):
        """Whether ``agk_wgrad`` takes these operands (asked before a push is attached to the preceding launch: a
        pushed epoch must be consumed)."""
        rows, K = x_local.shape
        T, N = dy.shape
        return (rows % 128 == 0 and rows * self.tp <= self.max_tokens and K <= self.hidden and K % 8 == 0
                and self._pair(rows, N) and T == rows * self.tp and N % 8 == 0 and K >= 256 and dw32 is not None
                and dw32.dtype == torch.float32 and dw32.is_contiguous() and tuple(dw32.shape) == (N, K)
                and x_local.is_contiguous())

    def agk_wgrad(self, dy, x_local, dw32):
        """``dw32 [N, K] += dyᵀ · gather(x_local)`` in one kernel (the gather runs along the reduction rows).
        When the preceding ``gemm_rs(..., push=x_local)`` already carried the push of ``x_local``, this launch only
        consumes the flagged rows.  Returns True, or None when the shape is unsupported."""
        from ..ops import cuda as cu
        rows, K = x_local.shape
        T, N = dy.shape
        if not self._ok("agk_wgrad", x_local, rows, K):
            return None
        if not self._pair(rows, N) or T != rows * self.tp or N % 8 or K < 256 or dw32.dtype != torch.float32 \
                or not dw32.is_contiguous() or tuple(dw32.shape) != (N, K):
            return self._refuse("agk_wgrad", x_local, "needs rows per rank a multiple of 256 and a contiguous fp32 [N, K] gradient")
        x_local = x_local.contiguous()
        dy = dy.contiguous()
        pushed = self._pushed is not None and self._pushed == (x_local.data_ptr(), rows, K, self.epoch_ag)
        self._pushed = None
        n_comm = 0 if pushed else self.n_comm_ag
        if pushed:      # same epoch and gathered buffer as the push
            ptrs = (self._arr(self.gathered_ptrs[self.epoch_ag & 1]), self._arr(self.ag_flags), self._arr(self.ag_done),
                    c_void_p(self.counters.data_ptr()), _u32(self.ag_count), c_int(_MAX_FLAGS))
        else:
            ptrs = self._ag_args()
        rc = cu.lib().ell_gemm_agk_wgrad_pair(cu._p(dy), cu._p(x_local), cu._p(dw32), c_int(rows), c_int(N), c_int(K),
                                              c_int(self.rank), c_int(self.tp), _u32(self.epoch_ag),
                                              c_int(n_comm), *ptrs, cu._p(cu.err_flag(dy.device)), cu._stream())
        self.ag_count += self.grid_pair - n_comm
        cu._check(rc, "gemm_agk_wgrad")
        self._last_ag = (x_local, rows, K, self._gathered_off[self.epoch_ag & 1])
        return True

    def gathered(self):
        """The all-gathered operand ``[T, K]`` of the last gather kernel (a view into the workspace, valid until the
        next fused call).  Peers' shards were pushed by the kernel; the local shard is copied in here."""
        x_local, rows, K, off = self._last_ag
        full = self.buf[off: off + rows * self.tp * K * 2].view(torch.bfloat16).view(rows * self.tp, K)
        full[self.rank * rows:(self.rank + 1) * rows].copy_(x_local)
        return full

    def gemm_rs(self, x, w, b_mn=False, all_reduce=False, push=None):
        """reduce-scatter over TP of ``x · op(w)``: this rank's ``[T/tp, N]`` rows; with ``all_reduce`` the full
        ``[T, N]`` sum on every rank.  None when the shape is unsupported.
        ``push``: a sequence shard ``[T/tp, K']`` whose all-gather the NEXT fused call (``agk_wgrad`` on the same
        tensor) needs: a few more CTAs of this launch copy it to the peers while the main loop runs."""
        from ..ops import cuda as cu
        op = "gemm_ar" if all_reduce else "gemm_rs"
        M, K = x.shape
        N = w.shape[1] if b_mn else w.shape[0]
        if M % self.tp:
            return self._refuse(op, x, f"{M} rows do not divide over {self.tp} ranks")
        rows = M // self.tp
        bn = 256 if N >= 256 else 128
        tiles_n = (N + bn - 1) // bn
        if not self._ok(op, x, rows, N):
            return None
        if N % bn or (rows // 128) * tiles_n > _MAX_FLAGS or K % 8:
            return self._refuse(op, x, f"N = {N} must be a multiple of {bn}, K = {K} of 8")
        x = x.contiguous()
        y = torch.empty(M if all_reduce else rows, N, dtype=torch.bfloat16, device=x.device)
        self.epoch_rs += 1
        lib = cu.lib()
        pair = self._pair(rows, N)
        n_comm = self._reduce_ctas(K)
        grid = self.grid_pair if pair else self.grid_single
        head = (cu._p(x), cu._p(w), cu._p(y), c_int(rows), c_int(N), c_int(K), c_int(1 if b_mn else 0),
                c_int(self.rank), c_int(self.tp), _u32(self.epoch_rs), c_int(n_comm),
                self._arr(self.stage_ptrs), self._arr(self.rs_flags), self._arr(self.red_flags), self._arr(self.rs_done),
                c_void_p(self.counters.data_ptr() + 8), _u32(self.rs_count), c_int(_MAX_FLAGS), _u32(self.rs_queue),
                c_int(1 if all_reduce else 0))
        tail = (cu._p(cu.err_flag(x.device)), cu._stream())
        n_push = 0
        self._pushed = None
        if pair:
            push_args = (c_void_p(0), c_int(0), c_int(0), c_uint(0), c_int(0), self._arr(self.gathered_ptrs[0]),
                         self._arr(self.ag_flags), self._arr(self.ag_done))
            if push is not None and push.dim() == 2 and push.shape[0] == rows and push.shape[1] % 8 == 0 \
                    and push.shape[1] <= self.hidden and push.is_contiguous() and self.tp > 1:
                self.epoch_ag += 1
                n_push = self.n_comm_ag
                push_args = (cu._p(push), c_int(rows), c_int(push.shape[1]), _u32(self.epoch_ag), c_int(n_push),
                             self._arr(self.gathered_ptrs[self.epoch_ag & 1]), self._arr(self.ag_flags),
                             self._arr(self.ag_done))
                self._pushed = (push.data_ptr(), rows, push.shape[1], self.epoch_ag)
            rc = lib.ell_gemm_rs_pair(*head, *push_args, *tail)
        else:
            rc = lib.ell_gemm_rs(*head, *tail)
        cu._check(rc, op)
        self.rs_count += grid - n_push
        if all_reduce or not pair:
            # the staged reduction hands tiles out through a queue that every CTA running the reduce role (all but
            # the push CTAs) overshoots by one; the CTA-pair reduce-scatter sums in its epilogue and has no queue
            self.rs_queue += lib.ell_gemm_rs_queue_advance(c_int(rows), c_int(N), c_int(self.tp),
                                                           c_int(1 if all_reduce else 0), c_int(grid - n_push))
        return y

    def ce_combine(self, parts):
        """Cross-rank combine of the per-token cross-entropy statistics ``parts [T, 3]`` = (max, sum-exp, target
        logit): every rank pushes its triple to the peers' workspace and merges what it received, in one kernel.
        Returns ``(lse [T], target_logit [T])`` or None."""
        from ..ops import cuda as cu
        T = parts.shape[0]
        if T > self.max_tokens or not cu.has_symbol("ell_ce_combine_tp"):
            return None
        parts = parts.contiguous()
        out = torch.empty(2, T, dtype=torch.float32, device=parts.device)
        self.epoch_ce += 1
        rc = cu.lib().ell_ce_combine_tp(cu._p(parts), cu._p(out), c_int(T), c_int(self.max_tokens), c_int(self.rank),
                                        c_int(self.tp), _u32(self.epoch_ce), self._arr(self.ce_bufs),
                                        self._arr(self.ce_flags), cu._p(cu.err_flag(parts.device)), cu._stream())
        cu._check(rc, "ce_combine_tp")
        return out[0], out[1]


_WS = None


def install(max_tokens, hidden, allow_single_rank=False):
    """Create the workspace for this TP group and route the TP linears through the fused kernels.
    ``allow_single_rank`` builds it for a one-rank group too (the kernels then run their whole flag, staging and
    reduce machinery without peers: used by single-GPU tests and profiler captures)."""
    global _WS
    from . import tp_linear
    g = get_grid()
    if (g.tp == 1 and not allow_single_rank) or not torch.cuda.is_available():
        return None
    _WS = FusedTPWorkspace(max_tokens, hidden)

    def ag(x, w, bias, b_mn=False, want_gathered=False):
        y = _WS.ag_gemm(x, w, bias, b_mn)
        if y is None:
            return None
        return (y, _WS.gathered() if want_gathered else None)

    def rs(x, w, b_mn=False, all_reduce=False, push=None):
        return _WS.gemm_rs(x, w, b_mn, all_reduce, push)

    def agk(dy, x, dw32, dry_run=False):
        return _WS.agk_accepts(dy, x, dw32) if dry_run else _WS.agk_wgrad(dy, x, dw32)

    tp_linear.set_fused_impl(ag, rs, agk)
    return _WS


def uninstall():
    global _WS
    from . import tp_linear
    tp_linear.set_fused_impl(None, None, None)
    _WS = None


def workspace():
    return _WS
