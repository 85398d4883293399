"""Differentiable hot ops of the framework.

Every op has two implementations with one signature:

* the sm_100a kernels of ``libeasyllm_b200.so`` (``ops.cuda``), used for CUDA bf16 tensors —
  the product path; a missing library on a GPU machine raises instead of falling back;
* the PyTorch statement in ``ops.reference`` — what runs on CPU (gloo tests, fp32 parity
  configs), the numerical oracle of the kernel tests, and, with ``set_backend("torch")``, the
  unfused library path used for A/B comparison on a GPU (cuBLAS matmul + library attention).

Weights may carry a ``main_grad`` attribute (an fp32 view into the engine's flat gradient
buffer).  When present, weight gradients are accumulated straight into it by the kernels
(wgrad GEMM with beta = 1, norm weight-gradient reduce) and autograd receives ``None``.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import reference as ref

_BACKEND = os.environ.get("EASYLLM_OPS", "b200")          # b200 | torch
_GEMM = os.environ.get("EASYLLM_GEMM", "tcgen05")         # tcgen05 | cublas
_ATTN = os.environ.get("EASYLLM_ATTN", "auto")            # auto | kernel | library
_STRICT = os.environ.get("EASYLLM_STRICT", "0") == "1"    # 1: a shape the kernels cannot take raises instead of falling back
_FALLBACKS = {}                                           # (op, reason) -> count, for reports and tests


def set_strict(flag):
    """With strict mode on, a CUDA bf16 call that cannot run on the sm_100a kernels raises instead of taking the
    PyTorch / library path (benchmarks run strict, so a lost product path cannot go unnoticed)."""
    global _STRICT
    _STRICT = bool(flag)


def fallbacks():
    """``{(op, reason): count}`` of the calls that left the kernel path since the process started."""
    return dict(_FALLBACKS)


def note_fallback(op, t, reason):
    """Record that a CUDA bf16 call of ``op`` takes the PyTorch / library path.  Logged once per (op, reason)
    with the offending shape; raises under strict mode.  CPU tensors, other dtypes and an explicitly selected
    ``torch`` / ``cublas`` backend are deliberate choices and are not reported."""
    if not (torch.is_tensor(t) and t.is_cuda and t.dtype == torch.bfloat16 and _BACKEND == "b200"):
        return
    msg = f"{op}: {reason} (shape {tuple(t.shape)}); taking the PyTorch / library path instead of the sm_100a kernel"
    if _STRICT:
        raise RuntimeError(msg + " [EASYLLM_STRICT=1]")
    key = (op, reason)
    if key not in _FALLBACKS:
        from ..utils.log import default_logger
        default_logger.warning(msg)
    _FALLBACKS[key] = _FALLBACKS.get(key, 0) + 1


def set_backend(name):
    global _BACKEND
    if name not in ("b200", "torch"):
        raise ValueError(name)
    _BACKEND = name


def get_backend():
    return _BACKEND


def set_gemm_backend(name):
    global _GEMM
    if name not in ("tcgen05", "cublas"):
        raise ValueError(name)
    _GEMM = name


def get_gemm_backend():
    return _GEMM


def set_attention_backend(name):
    global _ATTN
    _ATTN = name


def _kern(x):
    return _BACKEND == "b200" and x.is_cuda and x.dtype == torch.bfloat16


def _cu():
    from . import cuda
    return cuda


def kernel_launches():
    from . import cuda
    return cuda.LAUNCHES


def _grad_to(param, g32):
    """Deliver an fp32 weight gradient: into ``param.main_grad`` (returns None) or as a tensor."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        mg.add_(g32.view_as(mg))
        return None
    return g32.to(param.dtype)


# ---------------------------------------------------------------------------------------------
# RMSNorm (+ residual add)
# ---------------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, _, rstd = _cu().rmsnorm_fwd(x, None, w, eps)
        ctx.save_for_backward(x, w, rstd)
        ctx.wref = w
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        mg = getattr(ctx.wref, "main_grad", None)
        if mg is not None:
            dx, _ = _cu().rmsnorm_bwd(dy.contiguous(), x, w, rstd, None, dw_out=mg, accumulate=True)
            return dx, None, None
        dx, dw = _cu().rmsnorm_bwd(dy.contiguous(), x, w, rstd)
        return dx, dw.to(w.dtype), None


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps):
        y, h, rstd = _cu().rmsnorm_fwd(x, residual, w, eps)
        ctx.save_for_backward(h, w, rstd)
        ctx.wref = w
        ctx.mark_non_differentiable()
        return y, h

    @staticmethod
    def backward(ctx, dy, dh_in):
        h, w, rstd = ctx.saved_tensors
        mg = getattr(ctx.wref, "main_grad", None)
        dres = dh_in.contiguous() if dh_in is not None else None
        if mg is not None:
            dh, _ = _cu().rmsnorm_bwd(dy.contiguous(), h, w, rstd, dres, dw_out=mg, accumulate=True)
            return dh, dh, None, None
        dh, dw = _cu().rmsnorm_bwd(dy.contiguous(), h, w, rstd, dres)
        return dh, dh, dw.to(w.dtype), None


def _norm_ok(x, op):
    if not _kern(x):
        return False
    if x.shape[-1] % 8 or x.shape[-1] > 8192:
        note_fallback(op, x, "the row length must be a multiple of 8 and at most 8192")
        return False
    return True


def rmsnorm(x, weight, eps=1e-6):
    if _norm_ok(x, "rmsnorm"):
        return _RMSNorm.apply(x.reshape(-1, x.shape[-1]).contiguous(), weight, eps).view(x.shape)
    return ref.rmsnorm(x, weight, eps)


def add_rmsnorm(x, residual, weight, eps=1e-6):
    """Returns (norm(x + residual), x + residual)."""
    if _norm_ok(x, "add_rmsnorm"):
        H = x.shape[-1]
        y, h = _AddRMSNorm.apply(x.reshape(-1, H).contiguous(), residual.reshape(-1, H).contiguous(), weight, eps)
        return y.view(x.shape), h.view(x.shape)
    return ref.add_rmsnorm(x, residual, weight, eps)


# ---------------------------------------------------------------------------------------------
# Affine LayerNorm (+ residual add), mixed precision
# ---------------------------------------------------------------------------------------------
class _LayerNorm(torch.autograd.Function):
    """LayerNorm(x (+ residual)) · w + b on the sm_100a kernel; parameter gradients in fp32, straight into
    ``main_grad`` when the parameters carry one."""

    @staticmethod
    def forward(ctx, x, residual, w, b, eps):
        y, h, mean, rstd = _cu().layernorm_fwd(x, residual, w, b, eps)
        ctx.save_for_backward(h, w, mean, rstd)
        ctx.refs = (w, b)
        ctx.has_res = residual is not None
        if residual is None:
            return y
        ctx.mark_non_differentiable()
        return y, h

    @staticmethod
    def backward(ctx, dy, dh_in=None):
        h, w, mean, rstd = ctx.saved_tensors
        wref, bref = ctx.refs
        mgw, mgb = getattr(wref, "main_grad", None), getattr(bref, "main_grad", None)
        direct = mgw is not None and mgb is not None
        dw = mgw if direct else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        db = mgb if direct else torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        dres = dh_in.contiguous() if (ctx.has_res and dh_in is not None) else None
        dh = _cu().layernorm_bwd(dy.contiguous(), h, w, mean, rstd, dres, dw, db)
        gw, gb = (None, None) if direct else (dw.to(w.dtype), db.to(w.dtype))
        return dh, (dh if ctx.has_res else None), gw, gb, None


def layernorm(x, weight, bias, eps=1e-5, residual=None):
    """Affine LayerNorm over the last dim with fp32 statistics.  With ``residual`` returns
    ``(norm(x + residual), x + residual)``."""
    if _kern(x):
        if x.shape[-1] % 8 == 0 and weight.dtype == torch.bfloat16:
            H = x.shape[-1]
            x2 = x.reshape(-1, H).contiguous()
            if residual is None:
                return _LayerNorm.apply(x2, None, weight, bias, eps).view(x.shape)
            y, h = _LayerNorm.apply(x2, residual.reshape(-1, H).contiguous(), weight, bias, eps)
            return y.view(x.shape), h.view(x.shape)
        note_fallback("layernorm", x, "the row length must be a multiple of 8 and the parameters bf16")
    h = x if residual is None else x + residual
    y = F.layer_norm(h.float(), h.shape[-1:], weight.float(), bias.float(), eps).to(h.dtype)
    return y if residual is None else (y, h)


# ---------------------------------------------------------------------------------------------
# Linear:  y = x · Wᵀ (+ b)
# ---------------------------------------------------------------------------------------------
def _gemm_ok(op, a, *dims):
    """tcgen05 GEMM eligibility: every row length and the output width must be a multiple of 8 elements (TMA
    strides are multiples of 16 bytes)."""
    if not _kern(a) or _GEMM != "tcgen05":
        return False
    if any(d % 8 for d in dims):
        note_fallback(op, a, f"dimensions {dims} must all be multiples of 8")
        return False
    return True


def matmul_nt(a, b, bias=None):
    """a [M,K] · b [N,K]ᵀ → [M,N] (bf16)."""
    if _gemm_ok("matmul_nt", a, a.shape[-1], b.shape[-1], b.shape[0]):
        return _cu().gemm(a, b, bias=bias)
    return F.linear(a, b, bias)


def matmul_nn(a, b):
    """a [M,K] · b [K,N] → [M,N]; b is read in place as an MN-major operand."""
    if _gemm_ok("matmul_nn", a, a.shape[-1], b.shape[-1]):
        return _cu().gemm(a, b, b_mn=True)
    return a @ b


def matmul_tn_accum(a, b, out32=None):
    """aᵀ [K,M]ᵀ·b [K,N] → [M,N] fp32, accumulated into ``out32`` when given."""
    if _gemm_ok("matmul_tn", a, a.shape[-1], b.shape[-1]):
        if out32 is None:
            return _cu().gemm(a, b, a_mn=True, b_mn=True, out_mode=2)
        return _cu().gemm(a, b, out=out32, a_mn=True, b_mn=True, out_mode=1)
    r = (a.t() @ b).float()
    if out32 is None:
        return r
    out32.add_(r)
    return out32


def column_sum(x):
    """fp32 column sums ``x.sum(0)`` of a 2-D tensor (the bias gradient of a linear layer)."""
    if _kern(x) and x.dim() == 2 and x.shape[1] % 8 == 0:
        out = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device)
        return _cu().colsum_(x.contiguous(), out)
    return x.float().sum(0)


def matmul_tn(a, b):
    """aᵀ [K,M]ᵀ·b [K,N] → [M,N] in the operands' dtype: a weight gradient handed to autograd (no fp32 ``main_grad``
    to accumulate into), rounded once in the GEMM epilogue."""
    if _gemm_ok("matmul_tn", a, a.shape[-1], b.shape[-1]):
        return _cu().gemm(a, b, a_mn=True, b_mn=True, out_mode=0)
    return a.t() @ b


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.wref, ctx.bref = w, bias
        return matmul_nt(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_nn(dy, w) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.wref, "main_grad", None)
            if mg is not None:
                matmul_tn_accum(dy, x, mg)
            else:
                dw = matmul_tn(dy, x)
        db = None
        if ctx.bref is not None and ctx.needs_input_grad[2]:
            db = _grad_to(ctx.bref, column_sum(dy))
        return dx, dw, db


def linear(x, w, bias=None):
    if _kern(x):
        y = _Linear.apply(x.reshape(-1, x.shape[-1]).contiguous(), w, bias)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])
    return F.linear(x, w, bias)


def _adjacent_alias(tensors):
    """One ``[sum(rows), cols]`` tensor aliasing ``tensors`` when they sit back to back in one storage (as the
    parameters of a module do after the optimizer moved them into its flat buffer), else None."""
    t0 = tensors[0]
    if not all(t.is_contiguous() and t.dim() == 2 and t.shape[1] == t0.shape[1] and t.dtype == t0.dtype for t in tensors):
        return None
    ptr, base = t0.data_ptr(), t0.untyped_storage().data_ptr()
    for t in tensors:
        # adjacent addresses are not enough: separate allocations can be neighbours in the caching allocator
        if t.data_ptr() != ptr or t.untyped_storage().data_ptr() != base:
            return None
        ptr += t.numel() * t.element_size()
    rows = sum(t.shape[0] for t in tensors)
    return torch.as_strided(t0, (rows, t0.shape[1]), (t0.shape[1], 1))


class _LinearParts(torch.autograd.Function):
    """``x · [W_1; W_2; ...]ᵀ`` for projections stored as separate parameters (q/k/v, gate/up of the HF-named
    modules).  When the parameters (and their fp32 ``main_grad`` views) are adjacent in memory the fused weight is
    an alias — nothing is concatenated, and the wgrad GEMM accumulates into the fused ``main_grad`` in one call."""

    @staticmethod
    def forward(ctx, x, bias, *weights):
        alias = _adjacent_alias([w.detach() for w in weights])
        W = alias if alias is not None else torch.cat([w.detach() for w in weights], 0)
        ctx.save_for_backward(x, W)
        ctx.wrefs = weights
        ctx.has_bias = bias is not None
        return matmul_nt(x, W, bias)

    @staticmethod
    def backward(ctx, dy):
        x, W = ctx.saved_tensors
        dy = dy.contiguous()
        dx = matmul_nn(dy, W) if ctx.needs_input_grad[0] else None
        db = column_sum(dy).to(dy.dtype) if ctx.has_bias and ctx.needs_input_grad[1] else None
        ws = ctx.wrefs
        if not any(ctx.needs_input_grad[2:]):
            return (dx, db) + (None,) * len(ws)
        mgs = [getattr(w, "main_grad", None) for w in ws]
        if all(m is not None for m in mgs):
            fused = _adjacent_alias(mgs)
            if fused is not None:
                matmul_tn_accum(dy, x, fused)
            else:
                r0 = 0
                for w, m in zip(ws, mgs):
                    matmul_tn_accum(dy[:, r0:r0 + w.shape[0]].contiguous(), x, m)
                    r0 += w.shape[0]
            return (dx, db) + (None,) * len(ws)
        dW = matmul_tn(dy, x)
        return (dx, db) + tuple(dW.split([w.shape[0] for w in ws], 0))


def linear_parts(x, weights, biases=None):
    """``x · concat(weights)ᵀ (+ concat(biases))`` without materialising the concatenation when avoidable."""
    bias = None
    if biases is not None and all(b is not None for b in biases):
        bias = torch.cat(list(biases), 0)
    if _kern(x):
        y = _LinearParts.apply(x.reshape(-1, x.shape[-1]).contiguous(), bias, *weights)
        return y if x.dim() == 2 else y.view(*x.shape[:-1], y.shape[-1])
    return F.linear(x, torch.cat(list(weights), 0), bias)


# ---------------------------------------------------------------------------------------------
# Vocab-parallel embedding lookup (partial: rows of ids owned by other ranks are zero)
# ---------------------------------------------------------------------------------------------
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, vocab_start, vocab_total):
        ctx.save_for_backward(ids)
        ctx.wref = weight
        ctx.start = vocab_start
        return _cu().embedding_fwd(ids, weight, vocab_start, vocab_total)

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        w = ctx.wref
        mg = getattr(w, "main_grad", None)
        dout = dout.contiguous()
        if mg is not None:
            _cu().embedding_bwd_(ids, dout, mg, ctx.start)
            return None, None, None, None
        g32 = torch.zeros(w.shape, dtype=torch.float32, device=w.device)
        _cu().embedding_bwd_(ids, dout, g32, ctx.start)
        return None, g32.to(w.dtype), None, None


def embedding(ids, weight, vocab_start=0, vocab_total=0):
    """``weight[ids - vocab_start]`` with zero rows for ids outside this rank's vocabulary range.  On the kernel
    path ``vocab_total`` turns on the device-side range check of the ids (error word, no host sync)."""
    if _kern(weight):
        if weight.shape[1] % 8 == 0 and weight.is_contiguous():
            return _Embedding.apply(ids, weight, vocab_start, vocab_total)
        note_fallback("embedding", weight, "the table must be contiguous with a row length that is a multiple of 8")
    rows = weight.shape[0]
    mask = (ids < vocab_start) | (ids >= vocab_start + rows)
    out = F.embedding((ids - vocab_start).masked_fill(mask, 0), weight)
    return out.masked_fill(mask.unsqueeze(-1), 0.0) if bool(mask.any()) else out


# ---------------------------------------------------------------------------------------------
# RoPE on the packed QKV rows, SwiGLU on the fused gate|up rows
# ---------------------------------------------------------------------------------------------
class _RopePacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, pos, n_rot_heads, head_dim):
        ctx.save_for_backward(cos, sin, pos)
        ctx.meta = (n_rot_heads, head_dim)
        _cu().rope_(qkv, cos, sin, pos, n_rot_heads, head_dim)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, g):
        cos, sin, pos = ctx.saved_tensors
        g = g.contiguous().clone() if not g.is_contiguous() else g.clone()
        _cu().rope_(g, cos, sin, pos, *ctx.meta, backward=True)
        return g, None, None, None, None, None


def rope_packed(qkv, cos, sin, pos, n_q_heads, n_kv_heads, head_dim):
    """Rotate the q and k heads of ``qkv [T, (Hq+2Hk)·D]`` (layout q|k|v) at positions ``pos``."""
    if _kern(qkv):
        if head_dim % 16 == 0:
            pos32 = pos if pos.dtype == torch.int32 else pos.to(torch.int32)
            return _RopePacked.apply(qkv, cos, sin, pos32, n_q_heads + n_kv_heads, head_dim)
        note_fallback("rope", qkv, f"head_dim {head_dim} must be a multiple of 16")
    T = qkv.shape[0]
    nq, nk = n_q_heads * head_dim, n_kv_heads * head_dim
    q = qkv[:, :nq].reshape(T, n_q_heads, head_dim)
    k = qkv[:, nq:nq + nk].reshape(T, n_kv_heads, head_dim)
    q, k = ref.rope(q, k, cos, sin, pos.long())
    return torch.cat((q.reshape(T, nq), k.reshape(T, nk), qkv[:, nq + nk:]), dim=1)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return _cu().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, d):
        (gu,) = ctx.saved_tensors
        return _cu().swiglu_bwd(d.contiguous(), gu)


def glu(gate_up, activation="silu"):
    """``act(gate) * up`` on fused rows ``[T, 2F]`` (gate columns first)."""
    if _kern(gate_up):
        if activation in ("silu", "swiglu") and gate_up.shape[-1] % 16 == 0:
            W = gate_up.shape[-1]
            return _SwiGLU.apply(gate_up.reshape(-1, W).contiguous()).view(*gate_up.shape[:-1], W // 2)
        note_fallback("glu", gate_up, f"activation {activation!r} / width must be silu and a multiple of 16")
    F_ = gate_up.shape[-1] // 2
    return ref.GLU_ACTIVATIONS[activation](gate_up[..., :F_], gate_up[..., F_:])


# ---------------------------------------------------------------------------------------------
# Attention
# ---------------------------------------------------------------------------------------------
def _library_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale):
    """cuDNN / library attention (counts as a library call, like cuBLAS)."""
    T, Hq, D = q.shape
    if cu_seqlens is None or cu_seqlens.numel() == 2:
        o = F.scaled_dot_product_attention(q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0),
                                           v.transpose(0, 1).unsqueeze(0), is_causal=causal, scale=scale,
                                           enable_gqa=k.shape[1] != Hq)
        return o.squeeze(0).transpose(0, 1).contiguous()
    cs = cu_seqlens.to(torch.int32)
    try:
        from torch.nn.attention.varlen import varlen_attn
        if causal:
            return varlen_attn(q, k, v, cs, cs, max_seqlen, max_seqlen, scale=scale, window_size=(-1, 0))
        return varlen_attn(q, k, v, cs, cs, max_seqlen, max_seqlen, scale=scale)
    except Exception:
        from flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func(q, k, v, cs, cs, max_seqlen, max_seqlen, softmax_scale=scale, causal=causal)


def _attn_kernel_reason(dtype, head_dim):
    """None when the sm_100a attention kernels take the call, else why not."""
    if _BACKEND != "b200" or _ATTN not in ("auto", "kernel"):
        return "backend"
    if dtype != torch.bfloat16:
        return "dtype"
    if head_dim > 128 or head_dim % 8:
        return f"head_dim {head_dim} (the kernels take up to 128, in multiples of 8)"
    return None


def _pad_heads(t, D):
    """[T, H, d] → [T, H, D] with zero columns: scores and outputs of the padded columns are exactly zero, so the
    128-wide kernels serve smaller heads (their tiles are half empty, which only small test models pay)."""
    return F.pad(t, (0, D - t.shape[-1]))


def flash_attention(q, k, v, cu_seqlens=None, max_seqlen=None, causal=True, scale=None, alibi_slopes=None):
    """Attention over packed documents: q ``[T,Hq,D]``, k/v ``[T,Hk,D]`` → ``[T,Hq,D]``.  ``alibi_slopes``
    (one per query head) adds ``slope · (key − query)`` to the scores.
    Pass ``max_seqlen`` (a Python int) with ``cu_seqlens``: deriving it here costs a device→host sync."""
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
        if max_seqlen is None:
            max_seqlen = q.shape[0] if cu_seqlens is None else int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        why = _attn_kernel_reason(q.dtype, D) or (None if causal else "non-causal")
        if why is None:
            if D < 128:
                o = _cu().flash_attention(_pad_heads(q, 128), _pad_heads(k, 128), _pad_heads(v, 128), cu_seqlens,
                                          max_seqlen, causal, scale, alibi_slopes)
                return o[..., :D]
            return _cu().flash_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale, alibi_slopes)
        if _ATTN == "kernel":
            raise RuntimeError(f"attention kernel does not support this call: {why}")
        if why not in ("backend", "dtype"):
            note_fallback("flash_attention", q, why)
        if alibi_slopes is None:
            return _library_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale)
    return ref.attention_varlen(q, k, v, cu_seqlens, causal, scale, alibi_slopes)


def flash_attention_packed(qkv, n_q_heads, n_kv_heads, head_dim, cu_seqlens=None, max_seqlen=None, scale=None,
                           alibi_slopes=None, rope=None, row_start=None):
    """(RoPE +) causal attention on the fused projection output ``qkv [T, (Hq+2Hk)·D]`` (layout q|k|v)
    → ``[T, Hq·D]``.  ``rope`` = (cos, sin, position_ids) rotates the q and k heads first.  ``row_start``
    (int32 ``[T]``, the first token of each token's document) may be passed when the caller has it, so it is built
    once per micro-batch and not once per layer.

    On the kernel path (head_dim 128) the rotation is in place and the backward writes one packed gradient."""
    T = qkv.shape[0]
    nq, nk = n_q_heads * head_dim, n_kv_heads * head_dim
    if scale is None:
        scale = 1.0 / math.sqrt(head_dim)
    if _kern(qkv) and qkv.dim() == 2 and head_dim == 128 and _attn_kernel_reason(qkv.dtype, head_dim) is None:
        qkv = qkv.contiguous()
        if max_seqlen is None:
            max_seqlen = T if cu_seqlens is None else int((cu_seqlens[1:] - cu_seqlens[:-1]).max())
        if rope is not None:
            cos, sin, pos = rope
            rope = (cos, sin, pos if pos.dtype == torch.int32 else pos.to(torch.int32))
        return _cu().flash_attention_packed(qkv, n_q_heads, n_kv_heads, head_dim, cu_seqlens, max_seqlen, scale, rope,
                                            row_start, alibi_slopes)
    if rope is not None:
        qkv = rope_packed(qkv, rope[0], rope[1], rope[2], n_q_heads, n_kv_heads, head_dim)
    q = qkv[:, :nq].view(T, n_q_heads, head_dim)
    k = qkv[:, nq:nq + nk].view(T, n_kv_heads, head_dim)
    v = qkv[:, nq + nk:].view(T, n_kv_heads, head_dim)
    return flash_attention(q, k, v, cu_seqlens, max_seqlen, True, scale, alibi_slopes).reshape(T, nq)


# ---------------------------------------------------------------------------------------------
# Vocab-parallel cross entropy (stand-alone and fused with the LM head)
# ---------------------------------------------------------------------------------------------
def _tp_info():
    from ..parallel.grid import get_grid
    g = get_grid()
    return g.tp_group, g.tp, g.tp_rank


def _tp_workspace():
    from ..parallel import symm
    return symm.workspace()


def _combine_parts(parts, group, tp):
    """Cross-rank combine of per-token ``parts [T, 3]`` = (max, sum-exp, target logit): returns (lse, target_logit).
    With the fused-TP workspace installed the exchange is one kernel over peer memory (3 floats per token and rank);
    otherwise a MAX and a SUM all-reduce."""
    mx, se, tl = parts[:, 0], parts[:, 1], parts[:, 2]
    if tp > 1:
        ws = _tp_workspace() if parts.is_cuda and _BACKEND == "b200" else None
        if ws is not None:
            res = ws.ce_combine(parts)
            if res is not None:
                return res
        gmx = mx.clone()
        dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=group)
        pair = torch.stack((se * torch.exp(mx - gmx), tl), dim=0)
        dist.all_reduce(pair, group=group)
        se, tl, mx = pair[0], pair[1], gmx
    return torch.log(se) + mx, tl


class _VocabParallelCE(torch.autograd.Function):
    """Per-token loss from vocab-parallel logits.  Parity with
    llm/models/mg_models/base_modules/functions/cross_entropy.py:22-112, including ``cut_size``
    (padded vocab tail on the last rank excluded)."""

    @staticmethod
    def forward(ctx, logits, target, cut_size, inplace_backward):
        group, tp, rank = _tp_info()
        Vp = logits.shape[-1]
        valid = Vp - cut_size if (cut_size and rank == tp - 1) else Vp
        start = rank * Vp
        flat = logits.reshape(-1, Vp)
        tflat = target.reshape(-1)
        if _kern(flat):
            flat = flat.contiguous()
            parts = _cu().ce_fwd(flat, tflat.contiguous(), start, valid)
        else:
            parts = torch.stack(ref.cross_entropy_parts(flat, tflat, start, valid), dim=1)
        lse, tl = _combine_parts(parts, group, tp)
        ctx.save_for_backward(flat, tflat, lse)
        ctx.meta = (start, valid, logits.shape, inplace_backward)
        return (lse - tl).view(target.shape)

    @staticmethod
    def backward(ctx, g):
        flat, tflat, lse = ctx.saved_tensors
        start, valid, shape, inplace = ctx.meta
        g = g.reshape(-1).float().contiguous()
        if _kern(flat):
            buf = flat if inplace else flat.clone()
            _cu().ce_bwd_(buf, tflat, lse, g, start, valid)
            return buf.view(shape), None, None, None
        lf = flat.float()
        p = torch.exp(lf - lse.unsqueeze(1))
        if valid < lf.shape[1]:
            p[:, valid:] = 0
        loc = tflat - start
        hit = (loc >= 0) & (loc < valid)
        rows = torch.nonzero(hit).squeeze(1)
        p[rows, loc[rows]] -= 1.0
        return (p * g.unsqueeze(1)).to(flat.dtype).view(shape), None, None, None


def vocab_parallel_cross_entropy(vocab_parallel_logits, target, cut_size=None, inplace_backward=False):
    return _VocabParallelCE.apply(vocab_parallel_logits, target, cut_size, inplace_backward)


class _LMHeadCE(torch.autograd.Function):
    """LM-head GEMM whose epilogue also produces the vocab-parallel cross-entropy statistics (row max,
    sum-exp, target logit) while each logits tile is still in registers; only 3 floats per token cross the
    TP group.  Backward turns the stored bf16 logits into dlogits in place, then runs dgrad and wgrad.
    Fuses llm/models/mg_models/base_modules/layers/lm_head.py:49-71 with
    llm/models/mg_models/base_modules/functions/cross_entropy.py:22-112."""

    @staticmethod
    def forward(ctx, hidden, weight, target, cut_size):
        group, tp, rank = _tp_info()
        Vp = weight.shape[0]
        valid = Vp - cut_size if (cut_size and rank == tp - 1) else Vp
        start = rank * Vp
        tflat = target.reshape(-1).contiguous()
        logits, parts = _cu().gemm_ce(hidden, weight, tflat, start, valid)
        lse, tl = _combine_parts(parts, group, tp)
        ctx.save_for_backward(hidden, weight, logits, tflat, lse)
        ctx.wref = weight
        ctx.meta = (start, valid)
        return (lse - tl).view(target.shape)

    @staticmethod
    def backward(ctx, g):
        hidden, weight, logits, tflat, lse = ctx.saved_tensors
        start, valid = ctx.meta
        dlogits = _cu().ce_bwd_(logits, tflat, lse, g.reshape(-1).float().contiguous(), start, valid)
        dx = matmul_nn(dlogits, weight) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(ctx.wref, "main_grad", None)
            if mg is not None:
                matmul_tn_accum(dlogits, hidden, mg)
            else:
                dw = matmul_tn(dlogits, hidden)
        return dx, dw, None, None


class _LMHeadCESP(torch.autograd.Function):
    """The LM head of a sequence-parallel model in three fused kernels: all-gather of the hidden rows → GEMM →
    cross-entropy statistics (forward), dlogits·W → reduce-scatter (input gradient) and all-gather → dlogitsᵀ·x
    (weight gradient).  Nothing is gathered by a separate collective (lm_head.py:53-57 of the reference gathers
    with ``gather_from_sequence_parallel_region`` first)."""

    @staticmethod
    def forward(ctx, x_local, weight, target, cut_size):
        group, tp, rank = _tp_info()
        ws = _tp_workspace()
        Vp = weight.shape[0]
        valid = Vp - cut_size if (cut_size and rank == tp - 1) else Vp
        start = rank * Vp
        tflat = target.reshape(-1).contiguous()
        logits, parts = ws.ag_gemm_ce(x_local, weight, tflat, start, valid)
        lse, tl = _combine_parts(parts, group, tp)
        ctx.save_for_backward(x_local, weight, logits, tflat, lse)
        ctx.wref = weight
        ctx.meta = (start, valid)
        return (lse - tl).view(target.shape)

    @staticmethod
    def backward(ctx, g):
        from ..parallel import mappings as mp
        x_local, weight, logits, tflat, lse = ctx.saved_tensors
        start, valid = ctx.meta
        ws = _tp_workspace()
        dlogits = _cu().ce_bwd_(logits, tflat, lse, g.reshape(-1).float().contiguous(), start, valid)
        dx = None
        mg = getattr(ctx.wref, "main_grad", None)
        if ctx.needs_input_grad[0]:
            can_push = mg is not None and ctx.needs_input_grad[1] and ws.agk_accepts(dlogits, x_local, mg)
            dx = ws.gemm_rs(dlogits, weight, b_mn=True, push=x_local if can_push else None)
            if dx is None:
                dx = mp.reduce_scatter_first_dim(matmul_nn(dlogits, weight))
        dw = None
        if ctx.needs_input_grad[1]:
            if mg is None or ws.agk_wgrad(dlogits, x_local, mg) is None:
                xg = mp.gather_first_dim(x_local)
                if mg is not None:
                    matmul_tn_accum(dlogits, xg, mg)
                else:
                    dw = matmul_tn(dlogits, xg)
        return dx, dw, None, None


def lm_head_cross_entropy(hidden, weight, target, cut_size=None, gather_sp=False):
    """LM head GEMM + vocab-parallel CE → per-token losses (fp32, shape of ``target``).  The bf16 logits
    live only between forward and backward; their buffer is overwritten by dlogits in backward.
    ``gather_sp``: ``hidden`` is this rank's sequence shard ``[T/tp, h]``; the gather over the TP group is part
    of the op (fused into the GEMM kernel when the fused-TP workspace is installed)."""
    if gather_sp:
        ws = _tp_workspace() if _kern(hidden) and _GEMM == "tcgen05" else None
        if ws is not None and hidden.dim() == 2 and ws._pair(hidden.shape[0], weight.shape[0]) \
                and hidden.shape[0] * ws.tp <= ws.max_tokens and hidden.shape[1] <= ws.hidden and weight.shape[0] % 8 == 0:
            return _LMHeadCESP.apply(hidden.contiguous(), weight, target, cut_size)
        if ws is not None:
            note_fallback("lm_head_cross_entropy", hidden, "the fused gather needs rows per rank in multiples of 256 "
                                                           "within the workspace")
        from ..parallel import mappings as mp
        hidden = mp.gather_from_sequence_parallel_region(hidden, True)
    if hidden.dim() == 2 and _gemm_ok("lm_head_cross_entropy", hidden, hidden.shape[1], weight.shape[0]):
        return _LMHeadCE.apply(hidden.contiguous(), weight, target, cut_size)
    logits = linear(hidden, weight)
    return vocab_parallel_cross_entropy(logits, target, cut_size, inplace_backward=True)


# ---------------------------------------------------------------------------------------------
# Fused Adam on flat buffers
# ---------------------------------------------------------------------------------------------
def fused_adam_(p32, g32, m, v, p_lowp, lr, betas, eps, weight_decay, step, adamw=True, grad_scale=1.0,
                scale_tensor=None, bias_correction=True):
    if p32.is_cuda and _BACKEND == "b200":
        _cu().adam(p32, g32, m, v, p_lowp, lr, betas[0], betas[1], eps, weight_decay, step, adamw, grad_scale,
                   scale_tensor, bias_correction)
        return
    gs = grad_scale * (float(scale_tensor) if scale_tensor is not None else 1.0)
    ref.adam_step(p32, g32, m, v, lr, betas[0], betas[1], eps, weight_decay, step, adamw, gs, bias_correction)
    if p_lowp is not None:
        p_lowp.copy_(p32)


def sumsq(x32):
    """Σ x² of an fp32 buffer as a 1-element fp32 tensor (no host sync)."""
    out = torch.zeros(1, dtype=torch.float32, device=x32.device)
    if x32.is_cuda and _BACKEND == "b200" and x32.dtype == torch.float32:
        _cu().sumsq(x32, out)
        return out
    return (x32.float() ** 2).sum().view(1)
