"""ctypes bridge to ``libeasyllm_b200.so`` (the in-tree sm_100a kernel library).

Each wrapper takes torch CUDA tensors, checks dtype / layout, and launches on the current
torch stream.  A missing library on a machine with a GPU is an error, never a silent
fallback: ``lib()`` raises with the build command.  ``LAUNCHES`` counts kernel launches of
this library (benchmarks report it).
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libeasyllm_b200.so")
_lib = None
LAUNCHES = 0
_err_flags = {}
_scratch = {}


class KernelError(RuntimeError):
    pass


def available():
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise KernelError(f"{_LIB_PATH} is missing: run `python -m easyllm_b200.ops.build` "
                              "(or __graft_entry__.build()) before using the CUDA ops")
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.ell_rmsnorm_bwd_scratch_elems.restype = c_longlong
    return _lib


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_tls = threading.local()


def _stream():
    """Current torch stream; also makes the device's context current on this thread for the
    library's own CUDA runtime (worker threads such as autograd's start without one)."""
    dev = torch.cuda.current_device()
    if getattr(_tls, "dev", None) != dev:
        rc = lib().ell_set_device(c_int(dev))
        if rc != 0:
            raise KernelError(f"cudaSetDevice({dev}) failed with code {rc}")
        _tls.dev = dev
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc, name):
    global LAUNCHES
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}"
                          + (f" ({torch.cuda.get_device_name()})" if rc > 0 else " (bad arguments)"))
    LAUNCHES += 1


def _bf16c(t, name):
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise TypeError(f"{name}: expected a CUDA bf16 tensor, got {t.dtype} on {t.device}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous")
    return t


def err_flag(device=None):
    """Per-device int32 word the kernels write when one of their bounded waits expires."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    f = _err_flags.get(dev)
    if f is None:
        f = torch.zeros(1, dtype=torch.int32, device=dev)
        _err_flags[dev] = f
    return f


def check_err_flag():
    """Synchronising read of the error word; raises if a kernel reported a timed-out wait."""
    f = err_flag()
    v = int(f.item())
    if v:
        f.zero_()
        raise KernelError(f"a kernel gave up a bounded wait (code {v}: 1 producer, 2 mma, 3 epilogue, 4 communication "
                          "role, 5 peer flag; 11-15 the same roles of the CTA-pair GEMM; 21 cross-entropy exchange; "
                          "31 a token id outside the embedding table; 32 a position outside the rotary tables; "
                          "6 / 16 a tile index outside a fused kernel's buffers)")


def waiting_kernels_in_use():
    """True once a kernel that waits on peers or on its own pipeline with a bounded wait has been given an error
    word in this process (the GEMM / attention kernels, the fused TP and ZeRO kernels)."""
    return bool(_err_flags)


def check_step_errors():
    """Once per optimizer step, before the update is applied: raise if any kernel of the step gave up a bounded
    wait (a peer that arrived later than the wait limit leaves a partially computed tile behind; the step must
    not be applied on top of it).  One device→host read; a no-op on machines without the kernel library."""
    if _err_flags and torch.cuda.is_available():
        check_err_flag()


def scratch(nelem, dtype=torch.float32, tag="default"):
    """Grow-only scratch buffer (per device, per tag) so hot ops do not allocate every call."""
    dev = torch.cuda.current_device()
    key = (dev, tag, dtype)
    b = _scratch.get(key)
    if b is None or b.numel() < nelem:
        b = torch.empty(max(int(nelem), 1), dtype=dtype, device=torch.device("cuda", dev))
        _scratch[key] = b
    return b


# ---- norm ------------------------------------------------------------------------------------
def rmsnorm_fwd(x, residual, w, eps):
    """Returns (y, h, rstd); h is x (+ residual) — the new residual stream — or x itself."""
    _bf16c(x, "x"); _bf16c(w, "weight")
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    h = torch.empty_like(x) if residual is not None else x
    if residual is not None:
        _bf16c(residual, "residual")
    rc = lib().ell_rmsnorm_fwd(_p(x), _p(residual), _p(w), _p(y), _p(h if residual is not None else None),
                               _p(rstd), c_int(rows), c_int(cols), c_float(eps), _stream())
    _check(rc, "rmsnorm_fwd")
    return y, h, rstd


def rmsnorm_bwd(dy, h, w, rstd, dres=None, dw_out=None, accumulate=False):
    """Returns (dh, dw fp32).  ``dres`` (grad arriving on the residual path) is added into dh."""
    _bf16c(dy, "dy"); _bf16c(h, "h")
    rows, cols = h.shape
    dh = torch.empty_like(h)
    dw = dw_out if dw_out is not None else torch.empty(cols, dtype=torch.float32, device=h.device)
    sc = scratch(lib().ell_rmsnorm_bwd_scratch_elems(c_int(rows), c_int(cols)), tag="rmsnorm_bwd")
    if dres is not None:
        _bf16c(dres, "dres")
    rc = lib().ell_rmsnorm_bwd(_p(dy), _p(h), _p(w), _p(rstd), _p(dres), _p(dh), _p(dw), _p(sc), c_int(rows),
                               c_int(cols), c_int(1 if accumulate else 0), _stream())
    _check(rc, "rmsnorm_bwd")
    global LAUNCHES
    LAUNCHES += 1  # the column reduce is a second launch
    return dh, dw


def layernorm_fwd(x, residual, w, b, eps):
    """Affine LayerNorm with fp32 statistics.  Returns (y, h, mean, rstd); h is x (+ residual) or x itself."""
    _bf16c(x, "x"); _bf16c(w, "weight"); _bf16c(b, "bias")
    rows, cols = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    h = torch.empty_like(x) if residual is not None else x
    if residual is not None:
        _bf16c(residual, "residual")
    rc = lib().ell_layernorm_fwd(_p(x), _p(residual), _p(w), _p(b), _p(y), _p(h if residual is not None else None),
                                 _p(mean), _p(rstd), c_int(rows), c_int(cols), c_float(eps), _stream())
    _check(rc, "layernorm_fwd")
    return y, h, mean, rstd


def layernorm_bwd(dy, h, w, mean, rstd, dres, dw32, db32):
    """Returns dh; the fp32 ``dw32`` / ``db32`` ``[cols]`` are accumulated into."""
    _bf16c(dy, "dy"); _bf16c(h, "h")
    rows, cols = h.shape
    dh = torch.empty_like(h)
    if dres is not None:
        _bf16c(dres, "dres")
    rc = lib().ell_layernorm_bwd(_p(dy), _p(h), _p(w), _p(mean), _p(rstd), _p(dres), _p(dh), _p(dw32), _p(db32),
                                 c_int(rows), c_int(cols), _stream())
    _check(rc, "layernorm_bwd")
    global LAUNCHES
    LAUNCHES += 1  # the parameter-gradient column pass is a second launch
    return dh


# ---- rope / swiglu ----------------------------------------------------------------------------
def rope_(qkv, cos, sin, pos, n_rot_heads, head_dim, backward=False):
    """In-place rotary embedding on the first ``n_rot_heads`` heads of each row of ``qkv [T, W]``."""
    _bf16c(qkv, "qkv")
    if pos.dtype != torch.int32:
        pos = pos.to(torch.int32)
    T, W = qkv.shape
    rc = lib().ell_rope(_p(qkv), _p(cos), _p(sin), _p(pos), c_int(T), c_int(W), c_int(n_rot_heads),
                        c_int(head_dim), c_int(1 if backward else 0), c_int(cos.shape[0]), _p(err_flag(qkv.device)),
                        _stream())
    _check(rc, "rope")
    return qkv


def swiglu_fwd(gu):
    _bf16c(gu, "gate_up")
    T, F2 = gu.shape
    out = torch.empty(T, F2 // 2, dtype=gu.dtype, device=gu.device)
    _check(lib().ell_swiglu_fwd(_p(gu), _p(out), c_int(T), c_int(F2 // 2), _stream()), "swiglu_fwd")
    return out


def swiglu_bwd(dout, gu):
    _bf16c(dout, "dout"); _bf16c(gu, "gate_up")
    T, F2 = gu.shape
    dgu = torch.empty_like(gu)
    _check(lib().ell_swiglu_bwd(_p(dout), _p(gu), _p(dgu), c_int(T), c_int(F2 // 2), _stream()), "swiglu_bwd")
    return dgu


def accum_bf16_to_f32(src, dst):
    _check(lib().ell_accum_bf16_to_f32(_p(src), _p(dst), c_longlong(src.numel()), _stream()), "accum")


def colsum_(x, out32):
    """``out32 [cols] += x.sum(0)`` for a bf16 matrix ``x [rows, cols]``, in fp32, without an fp32 copy of ``x``."""
    _bf16c(x, "x")
    rows, cols = x.shape
    _check(lib().ell_colsum_bf16(_p(x), _p(out32), c_int(rows), c_int(cols), _stream()), "colsum")
    return out32


# ---- optimizer --------------------------------------------------------------------------------
def adam(p, g, m, v, p_lowp, lr, beta1, beta2, eps, weight_decay, step, adamw=True, grad_scale=1.0,
         scale_ptr=None, bias_correction=True):
    c1 = 1.0 - beta1 ** step if bias_correction else 1.0
    c2 = 1.0 - beta2 ** step if bias_correction else 1.0
    rc = lib().ell_adam(_p(p), _p(g), _p(m), _p(v), _p(p_lowp), c_longlong(p.numel()), c_float(lr), c_float(beta1),
                        c_float(beta2), c_float(eps), c_float(weight_decay), c_float(c1), c_float(c2),
                        c_float(grad_scale), c_int(1 if adamw else 0), _p(scale_ptr), _stream())
    _check(rc, "adam")


def sumsq(x, out):
    _check(lib().ell_sumsq(_p(x), c_longlong(x.numel()), _p(out), _stream()), "sumsq")


# ---- embedding ----------------------------------------------------------------------------
def embedding_fwd(ids, weight, vocab_start, vocab_total=0):
    """Rows of ``weight [rows, h]`` for the ids in ``[vocab_start, vocab_start+rows)``, zeros for the others.
    With ``vocab_total`` an id outside ``[0, vocab_total)`` sets the device error word (read once per step by
    ``check_step_errors``) instead of being checked on the host."""
    _bf16c(weight, "weight")
    flat = ids.reshape(-1).contiguous()
    if flat.dtype != torch.int64:
        flat = flat.to(torch.int64)
    out = torch.empty(flat.numel(), weight.shape[1], dtype=torch.bfloat16, device=weight.device)
    rc = lib().ell_embedding_fwd(_p(flat), _p(weight), _p(out), c_int(flat.numel()), c_int(weight.shape[1]),
                                 c_longlong(vocab_start), c_longlong(weight.shape[0]), c_longlong(vocab_total),
                                 _p(err_flag(weight.device)), _stream())
    _check(rc, "embedding_fwd")
    return out.view(*ids.shape, weight.shape[1])


def embedding_bwd_(ids, dout, grad32, vocab_start):
    """``grad32[id - vocab_start] += dout[t]`` (fp32, in place) for the ids this rank owns."""
    flat = ids.reshape(-1).contiguous()
    if flat.dtype != torch.int64:
        flat = flat.to(torch.int64)
    d = dout.reshape(flat.numel(), -1)
    _bf16c(d, "dout")
    rc = lib().ell_embedding_bwd(_p(flat), _p(d), _p(grad32), c_int(flat.numel()), c_int(d.shape[1]),
                                 c_longlong(vocab_start), c_longlong(grad32.shape[0]), _stream())
    _check(rc, "embedding_bwd")


# ---- cross entropy ----------------------------------------------------------------------------
def ce_fwd(logits, target, vocab_start, valid_cols):
    _bf16c(logits, "logits")
    T, V = logits.shape
    parts = torch.empty(T, 3, dtype=torch.float32, device=logits.device)
    rc = lib().ell_ce_fwd(_p(logits), _p(target), _p(parts), c_int(T), c_int(V), c_int(valid_cols),
                          c_longlong(vocab_start), _stream())
    _check(rc, "ce_fwd")
    return parts


def ce_bwd_(logits, target, lse, scale, vocab_start, valid_cols):
    T, V = logits.shape
    rc = lib().ell_ce_bwd(_p(logits), _p(target), _p(lse), _p(scale), c_int(T), c_int(V), c_int(V),
                          c_int(valid_cols), c_longlong(vocab_start), _stream())
    _check(rc, "ce_bwd")
    return logits


# ---- GEMM -------------------------------------------------------------------------------------
_GEMM_PAIR = os.environ.get("ELL_GEMM_PAIR", "1") != "0"


def gemm_pair_enabled():
    return _GEMM_PAIR


def set_gemm_pair(enabled):
    """Switch for the CTA-pair GEMM (``csrc/gemm_pair.cu``: tcgen05.mma.cta_group::2, one 256 x 256 tile per
    two-CTA cluster, 7-14 % faster than the single-CTA kernel on the Llama shapes measured on B200).  On by
    default (``ELL_GEMM_PAIR=0`` turns it off); ``gemm`` uses it for plain launches without a tile-width hint
    whose output has at least one full 256 x 256 tile and whose row count fills the second CTA's half."""
    global _GEMM_PAIR
    _GEMM_PAIR = bool(enabled)


# launch-time refusals of a cluster launch (nothing ran, the error is not sticky): cannot co-schedule (-20), invalid
# configuration (9), launch out of resources (701), invalid cluster size (912)
_PAIR_LAUNCH_REFUSED = (-20, 9, 701, 912)


def _use_pair(M, N, bn):
    return _GEMM_PAIR and bn == 0 and M >= 256 and N >= 256 and (M % 256 == 0 or M >= 2048)


def gemm(a, b, out=None, bias=None, a_mn=False, b_mn=False, out_mode=0, bn=0, pair=None):
    """``C = op(A) · op(B)ᵀ`` on tcgen05.  K-major operands are row-major ``[rows, K]``; MN-major
    operands are row-major ``[K, rows]``.  out_mode 0: bf16 C; 1: fp32 C += ; 2: fp32 C =.
    ``pair`` forces (True) or forbids (False) the CTA-pair kernel; None lets the shape decide."""
    _bf16c(a, "a"); _bf16c(b, "b")
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: reduction dims differ ({K} vs {Kb})")
    if (a.shape[1] % 8) or (b.shape[1] % 8) or (N % 8):
        raise ValueError("gemm: row lengths must be multiples of 8 elements (16-byte TMA strides)")
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16 if out_mode == 0 else torch.float32, device=a.device)
    want = torch.bfloat16 if out_mode == 0 else torch.float32
    if out.dtype != want or not out.is_contiguous() or tuple(out.shape) != (M, N):
        raise ValueError("gemm: bad output tensor")
    if _use_pair(M, N, bn) if pair is None else pair:
        rc = lib().ell_gemm_bf16_pair(_p(a), _p(b), _p(out), _p(bias), c_int(M), c_int(N), c_int(K), c_int(a.shape[1]),
                                      c_int(b.shape[1]), c_int(N), c_int(1 if a_mn else 0), c_int(1 if b_mn else 0),
                                      c_int(out_mode), _p(err_flag(a.device)), _stream())
        if rc not in _PAIR_LAUNCH_REFUSED:
            _check(rc, "gemm_bf16_pair")
            return out
        # the launch itself was refused (no device work was issued): this device cannot co-schedule the two-CTA
        # cluster with the kernel's shared memory.  Use the single-CTA kernel from here on.
        import warnings
        warnings.warn(f"CTA-pair GEMM launch refused (code {rc}); using the single-CTA tcgen05 kernel")
        set_gemm_pair(False)
    rc = lib().ell_gemm_bf16(_p(a), _p(b), _p(out), _p(bias), c_int(M), c_int(N), c_int(K), c_int(a.shape[1]),
                             c_int(b.shape[1]), c_int(N), c_int(1 if a_mn else 0), c_int(1 if b_mn else 0),
                             c_int(out_mode), c_int(bn), _p(err_flag(a.device)), _stream())
    _check(rc, "gemm_bf16")
    return out


def flash_fwd_plan(row_start):
    """Host-only: per (tile pair, tile) of the attention forward the first key row, the number of 128-key tiles it
    walks and which of them are masked element-wise, from the kernel's own arithmetic (``row_start``: a list or CPU
    int32 tensor with the document start of every token).  Returns ``[(kv_lo, n_tiles, mask_bits), ...]``."""
    rs = [int(x) for x in row_start]
    T = len(rs)
    arr = (c_int * T)(*rs)
    n_pairs = (T + 255) // 256
    out = (c_int * (6 * n_pairs))()
    lib().ell_flash_fwd_plan(arr, c_int(T), out)
    return [tuple(out[3 * i:3 * i + 3]) for i in range(2 * n_pairs)]


def gemm_work_units(M, N, bn=256, fuse=0, tp=1, rank=0, ctas=148, allow_split=True):
    """Host-only: the (row tile, column tile, first column, width) work units of a single-CTA GEMM launch in the
    order the kernel walks them, produced by the kernel's own tile-order code (no GPU is touched).
    ``fuse``: 0 plain, 1 all-gather→GEMM, 2 GEMM→reduce-scatter."""
    cap = 2 * ((M + 127) // 128) * ((N + bn - 1) // bn) + 8
    buf = (c_int * (4 * cap))()
    n = lib().ell_gemm_enumerate_units(c_int(M), c_int(N), c_int(bn), c_int(fuse), c_int(tp), c_int(rank),
                                       c_int(ctas), c_int(1 if allow_split else 0), buf, c_int(cap))
    if n < 0:
        raise KernelError(f"gemm_work_units failed with code {n}")
    return [tuple(buf[4 * i:4 * i + 4]) for i in range(n)]


def gemm_pair_tiles(M, N):
    """Host-only: the (row tile, column tile) order of the CTA-pair GEMM's 256 x 256 tiles."""
    cap = ((M + 255) // 256) * ((N + 255) // 256)
    buf = (c_int * (2 * max(cap, 1)))()
    n = lib().ell_gemm_pair_enumerate_tiles(c_int(M), c_int(N), buf, c_int(cap))
    if n < 0:
        raise KernelError(f"gemm_pair_tiles failed with code {n}")
    return [tuple(buf[2 * i:2 * i + 2]) for i in range(n)]


def gemm_pair_units(M, N, resident=74, allow_split=True, fuse=0, tp=1, rank=0, n_comm=0):
    """Host-only: the (row tile, column tile, first column, width) work units of a CTA-pair GEMM launch on a device
    where ``resident`` two-CTA clusters fit, in the order the kernel walks them (unit ``u`` runs on cluster
    ``u % clusters``).  Returns ``(clusters, units)``; an under-filled last wave shows up as 128-wide units.
    ``fuse``: 0 plain, 1 all-gather→GEMM, 2 GEMM→reduce-scatter, 3 GEMM→all-reduce, 4 gather of the reduction
    rows; fused launches run on ``resident - n_comm / 2`` GEMM clusters."""
    tiles = ((M + 255) // 256) * ((N + 255) // 256)
    if fuse:
        clusters = resident - n_comm // 2
    else:
        lib().ell_gemm_set_tail_split(c_int(1 if allow_split else 0))
        try:
            clusters = lib().ell_gemm_pair_launch_clusters(c_int(tiles), c_int(resident))
        finally:
            lib().ell_gemm_set_tail_split(c_int(1))
    cap = 2 * tiles + 2
    buf = (c_int * (4 * cap))()
    n = lib().ell_gemm_pair_enumerate_units(c_int(M), c_int(N), c_int(clusters), c_int(1 if allow_split else 0),
                                            c_int(fuse), c_int(tp), c_int(rank), buf, c_int(cap))
    if n < 0:
        raise KernelError(f"gemm_pair_units failed with code {n}")
    return clusters, [tuple(buf[4 * i:4 * i + 4]) for i in range(n)]


def reduce_tile_order(rows_per_rank, tiles_n, tp, pair=True):
    """Host-only: the order in which the reduce role of the fused GEMM→reduce-scatter kernels takes the 128-row
    tiles a rank owns: ``[(row tile inside the shard, column tile), ...]`` by queue position."""
    cap = (rows_per_rank // 128) * tiles_n
    buf = (c_int * (2 * max(cap, 1)))()
    n = lib().ell_gemm_owned_tile_order(c_int(rows_per_rank), c_int(tiles_n), c_int(tp), c_int(1 if pair else 0), buf,
                                        c_int(cap))
    if n < 0:
        raise KernelError(f"reduce_tile_order failed with code {n}")
    return [tuple(buf[2 * i:2 * i + 2]) for i in range(n)]


def gemm_ce(x, w, target, vocab_start, valid_cols, pair=None):
    """LM-head GEMM with the cross-entropy statistics fused into its epilogue.

    Returns ``(logits [T, V] bf16, parts [T, 3] fp32)`` with parts = (row max, Σ exp(l − max), target logit or 0)
    over the first ``valid_cols`` columns — the same triple ``ce_fwd`` computes from stored logits."""
    _bf16c(x, "x"); _bf16c(w, "w")
    T, K = x.shape
    V = w.shape[0]
    if K % 8 or V % 8:
        raise ValueError("gemm_ce: K and V must be multiples of 8")
    logits = torch.empty(T, V, dtype=torch.bfloat16, device=x.device)
    use_pair = _use_pair(T, V, 0) if pair is None else pair
    tiles = lib().ell_gemm_ce_slots_pair(c_int(V)) if use_pair else lib().ell_gemm_ce_tiles(c_int(V))
    part = scratch(tiles * 3 * T, tag="gemm_ce_part")
    parts = torch.empty(T, 3, dtype=torch.float32, device=x.device)
    tgt = target if target.dtype == torch.int64 else target.to(torch.int64)
    fn = lib().ell_gemm_ce_pair if use_pair else lib().ell_gemm_ce
    rc = fn(_p(x), _p(w), _p(logits), _p(tgt.contiguous()), _p(part), c_int(T), c_int(V), c_int(K),
            c_longlong(vocab_start), c_int(valid_cols), _p(err_flag(x.device)), _stream())
    _check(rc, "gemm_ce")
    rc = lib().ell_ce_combine(_p(part), _p(parts), c_int(tiles), c_int(T), _stream())
    _check(rc, "ce_combine")
    return logits, parts


def has_symbol(name):
    try:
        getattr(lib(), name)
        return True
    except AttributeError:
        return False


# ---- flash attention -------------------------------------------------------------------------
_zero_rows = {}


def _row_start(cu_seqlens, T, device):
    """Document start of every token (int32 [T]): what the attention kernels mask with.  Models compute it once
    per micro-batch (``row_start_of``) and pass it down; this is the per-call fallback."""
    if cu_seqlens is None:
        z = _zero_rows.get((device, T))
        if z is None:
            z = _zero_rows[(device, T)] = torch.zeros(T, dtype=torch.int32, device=device)
        return z
    cu = cu_seqlens.to(device=device, dtype=torch.int64)
    return torch.repeat_interleave(cu[:-1], cu[1:] - cu[:-1], output_size=T).to(torch.int32)


def row_start_of(cu_seqlens, T, device):
    """``row_start[t]`` = first token of the document token ``t`` belongs to, from ``cu_seqlens`` (None: one
    document).  Built on the host when ``cu_seqlens`` is a CPU tensor (no device synchronisation)."""
    if cu_seqlens is not None and not cu_seqlens.is_cuda:
        cu = cu_seqlens.to(torch.int64)
        rs = torch.repeat_interleave(cu[:-1], cu[1:] - cu[:-1])
        if rs.numel() != T:
            raise ValueError(f"cu_seqlens cover {rs.numel()} tokens, the batch has {T}")
        return rs.to(torch.int32).to(device, non_blocking=True)
    return _row_start(cu_seqlens, T, device)


def _slopes(alibi_slopes, Hq, device):
    if alibi_slopes is None:
        return None
    sl = alibi_slopes.to(device=device, dtype=torch.float32).contiguous()
    if sl.numel() != Hq:
        raise ValueError(f"alibi_slopes must hold one slope per query head ({Hq}), got {sl.numel()}")
    return sl


def flash_attn_fwd(q, k, v, row_start, scale, alibi_slopes=None):
    """q [T,Hq,128], k/v [T,Hk,128] (last two dims contiguous, any row stride) → (out, lse [Hq,T]).
    ``alibi_slopes`` fp32 [Hq]: adds ``slope_h · (key − query)`` to the scores."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        if t.dtype != torch.bfloat16 or t.stride(2) != 1 or t.stride(1) != D:
            raise ValueError(f"flash_attn_fwd: {n} must be bf16 with contiguous [heads, 128] rows")
    if D != 128 or k.stride(0) != v.stride(0):
        raise ValueError("flash_attn_fwd: head_dim must be 128 and k/v must share a row stride")
    out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(Hq, T, dtype=torch.float32, device=q.device)
    sl = _slopes(alibi_slopes, Hq, q.device)
    rc = lib().ell_flash_attn_fwd(_p(q), _p(k), _p(v), _p(out), _p(lse), _p(row_start), c_int(T), c_int(Hq), c_int(Hk),
                                  c_int(q.stride(0)), c_int(k.stride(0)), c_float(scale), _p(sl),
                                  _p(err_flag(q.device)), _stream())
    _check(rc, "flash_attn_fwd")
    return out, lse


def flash_attn_bwd(do, q, k, v, out, lse, row_start, scale, dq=None, dk=None, dv=None, alibi_slopes=None):
    """Gradients of the causal attention.  ``dq/dk/dv`` may be views into one packed ``[T, (Hq+2Hk)·128]``
    buffer (row stride shared by dk and dv); they are allocated (contiguous) when not given."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    if not has_symbol("ell_flash_attn_bwd"):
        raise RuntimeError("libeasyllm_b200.so was built without ell_flash_attn_bwd")
    do = do.contiguous()
    out = out.contiguous()
    if dq is None:
        dq = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=q.device)
        dk = torch.empty(T, Hk, D, dtype=torch.bfloat16, device=q.device)
        dv = torch.empty(T, Hk, D, dtype=torch.bfloat16, device=q.device)
    if dk.stride(0) != dv.stride(0):
        raise ValueError("flash_attn_bwd: dk and dv must share a row stride")
    acc = scratch(T * Hq * D, tag="fa_bwd_dq")
    delta = scratch(T * Hq, tag="fa_bwd_delta")
    kv_acc = scratch(2 * T * Hk * D, tag="fa_bwd_dkv") if Hq > Hk else None
    rc = lib().ell_flash_attn_bwd(_p(q), _p(k), _p(v), _p(out), _p(do), _p(lse), _p(row_start), _p(dq), _p(dk), _p(dv),
                                  _p(acc), _p(delta), _p(kv_acc), c_int(T), c_int(Hq), c_int(Hk), c_int(q.stride(0)),
                                  c_int(k.stride(0)), c_int(dq.stride(0)), c_int(dk.stride(0)), c_float(scale),
                                  _p(_slopes(alibi_slopes, Hq, q.device)), _p(err_flag(q.device)), _stream())
    _check(rc, "flash_attn_bwd")
    global LAUNCHES
    LAUNCHES += 3  # memset, delta and dq-convert launches beside the main kernel
    return dq, dk, dv


_FA_BWD = "kernel"   # "kernel": tcgen05 backward; "library": differentiate the library attention


def set_attention_backward(which):
    global _FA_BWD
    assert which in ("kernel", "library")
    _FA_BWD = which


def _library_bwd(q, k, v, do, cu, has_cu, max_seqlen, scale):
    from . import _library_attention
    with torch.enable_grad():
        qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
        o = _library_attention(qq, kk, vv, cu if has_cu else None, max_seqlen, True, scale)
        return torch.autograd.grad(o, (qq, kk, vv), do)


class _FlashAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, scale, slopes):
        T = q.shape[0]
        rs = _row_start(cu_seqlens, T, q.device)
        out, lse = flash_attn_fwd(q, k, v, rs, scale, slopes)
        ctx.save_for_backward(q, k, v, out, lse, rs, cu_seqlens if cu_seqlens is not None else torch.empty(0))
        ctx.meta = (max_seqlen, scale, cu_seqlens is not None)
        ctx.slopes = slopes
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse, rs, cu = ctx.saved_tensors
        max_seqlen, scale, has_cu = ctx.meta
        if _FA_BWD == "kernel" or ctx.slopes is not None:
            dq, dk, dv = flash_attn_bwd(do, q, k, v, out, lse, rs, scale, alibi_slopes=ctx.slopes)
        else:
            dq, dk, dv = _library_bwd(q, k, v, do, cu, has_cu, max_seqlen, scale)
        return dq, dk, dv, None, None, None, None


def _split_packed(qkv, hq, hk, D):
    T = qkv.shape[0]
    nq, nk = hq * D, hk * D
    return (qkv[:, :nq].view(T, hq, D), qkv[:, nq:nq + nk].view(T, hk, D), qkv[:, nq + nk:].view(T, hk, D))


class _FlashAttnPacked(torch.autograd.Function):
    """(RoPE +) attention on the fused projection output ``qkv [T, (Hq+2Hk)·D]`` (layout q|k|v).

    The rotation is applied to ``qkv`` in place (the projection's backward does not need its output), and the
    backward writes dq, dk and dv straight into one packed gradient and un-rotates it in place, so neither
    slice gradients nor a copy for the rotary backward are materialised."""

    @staticmethod
    def forward(ctx, qkv, hq, hk, D, cu_seqlens, max_seqlen, scale, cos, sin, pos, row_start, slopes):
        T = qkv.shape[0]
        rs = row_start if row_start is not None else _row_start(cu_seqlens, T, qkv.device)
        if cos is not None:
            rope_(qkv, cos, sin, pos, hq + hk, D)
        q, k, v = _split_packed(qkv, hq, hk, D)
        ctx.slopes = slopes
        out, lse = flash_attn_fwd(q, k, v, rs, scale, slopes)
        none = torch.empty(0)
        ctx.save_for_backward(qkv, out, lse, rs, cu_seqlens if cu_seqlens is not None else none,
                              *((cos, sin, pos) if cos is not None else (none, none, none)))
        ctx.meta = (hq, hk, D, max_seqlen, scale, cu_seqlens is not None, cos is not None)
        return out.view(T, hq * D)

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse, rs, cu, cos, sin, pos = ctx.saved_tensors
        hq, hk, D, max_seqlen, scale, has_cu, has_rope = ctx.meta
        T = qkv.shape[0]
        q, k, v = _split_packed(qkv, hq, hk, D)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _split_packed(dqkv, hq, hk, D)
        do = do.reshape(T, hq, D)
        if _FA_BWD == "kernel" or ctx.slopes is not None:
            flash_attn_bwd(do, q, k, v, out, lse, rs, scale, dq, dk, dv, alibi_slopes=ctx.slopes)
        else:
            gq, gk, gv = _library_bwd(q, k, v, do, cu, has_cu, max_seqlen, scale)
            dq.copy_(gq); dk.copy_(gk); dv.copy_(gv)
        if has_rope:
            rope_(dqkv, cos, sin, pos, hq + hk, D, backward=True)
        return (dqkv,) + (None,) * 11


def flash_attention_packed(qkv, hq, hk, D, cu_seqlens, max_seqlen, scale, rope=None, row_start=None,
                           alibi_slopes=None):
    cos, sin, pos = rope if rope is not None else (None, None, None)
    return _FlashAttnPacked.apply(qkv, hq, hk, D, cu_seqlens, max_seqlen, scale, cos, sin, pos, row_start,
                                  alibi_slopes)


def flash_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale, alibi_slopes=None):
    if not causal:
        raise ValueError("the attention kernel is causal-only")
    return _FlashAttn.apply(q, k, v, cu_seqlens, max_seqlen, scale, alibi_slopes)
