"""Plain PyTorch statements of every hot op.

These are (a) what runs on CPU (gloo tests, tiny fp32 parity configs), (b) the numerical
oracle the sm_100a kernels are tested against, and (c) the op sequence of the unfused A/B
path.  Layout convention everywhere: activations are token-major 2-D ``[T, hidden]`` with
``T = batch · seq`` (packed; document boundaries in ``cu_seqlens``), heads as
``[T, heads, head_dim]``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x, weight, eps=1e-6):
    """``x · rsqrt(mean(x²) + eps) · w`` with fp32 statistics; output in x.dtype."""
    xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    return (xf * torch.rsqrt(var + eps) * weight.float()).to(x.dtype)


def add_rmsnorm(x, residual, weight, eps=1e-6):
    """(norm(x + residual), x + residual): the pre-norm block's residual add folded in."""
    h = (x.float() + residual.float()).to(x.dtype)
    return rmsnorm(h, weight, eps), h


def rotate_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def rope_tables(head_dim, max_pos, base=10000.0, scale_factor=1.0, device=None, ntk_max_pos=None):
    """fp32 cos/sin tables ``[max_pos, head_dim/2]`` (NeoX half-rotation convention).

    ``scale_factor`` is linear position scaling; ``ntk_max_pos`` switches on dynamic-NTK base
    stretching when ``max_pos`` exceeds it (positional_embeddings.py:39-89).
    """
    if ntk_max_pos is not None and max_pos > ntk_max_pos:
        base = base * ((scale_factor * max_pos / ntk_max_pos) - (scale_factor - 1)) ** (head_dim / (head_dim - 2))
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    t = torch.arange(max_pos, dtype=torch.float32, device=device) / scale_factor
    fr = torch.outer(t, inv)
    return fr.cos(), fr.sin()


def rope(q, k, cos, sin, position_ids):
    """Apply rotary embedding to ``q [T,Hq,D]`` and ``k [T,Hk,D]``; ``position_ids [T]`` int."""
    c = cos[position_ids].unsqueeze(1)
    s = sin[position_ids].unsqueeze(1)
    c = torch.cat((c, c), -1)
    s = torch.cat((s, s), -1)

    def ap(x):
        xf = x.float()
        return (xf * c + rotate_half(xf) * s).to(x.dtype)
    return ap(q), ap(k)


def swiglu(gate, up):
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


GLU_ACTIVATIONS = {
    "silu": lambda g, u: (F.silu(g.float()) * u.float()).to(g.dtype),
    "swiglu": lambda g, u: (F.silu(g.float()) * u.float()).to(g.dtype),
    "geglu": lambda g, u: (F.gelu(g.float()) * u.float()).to(g.dtype),
    "reglu": lambda g, u: (F.relu(g.float()) * u.float()).to(g.dtype),
    "liglu": lambda g, u: (g.float() * u.float()).to(g.dtype),
}


class _BiasGelu(torch.autograd.Function):
    """tanh-approximated GeLU of ``x + bias`` with its analytic backward (one fused elementwise pass each way).
    Parity: llm/models/mg_models/base_modules/layers/fused_bias_gelu.py:32-64 (unused by the Llama family)."""

    @staticmethod
    def forward(ctx, x, bias):
        ctx.save_for_backward(x, bias)
        y = (x + bias).float()
        return (y * 0.5 * (1.0 + torch.tanh(0.79788456 * y * (1 + 0.044715 * y * y)))).to(x.dtype)

    @staticmethod
    def backward(ctx, g):
        x, bias = ctx.saved_tensors
        y = (x + bias).float()
        t = torch.tanh(0.79788456 * y * (1 + 0.044715 * y * y))
        ff = 0.5 * y * ((1 - t * t) * (0.79788456 + 0.1070322243 * y * y)) + 0.5 * (1 + t)
        gx = (ff * g.float()).to(x.dtype)
        return gx, gx.reshape(-1, bias.shape[-1]).sum(0).to(bias.dtype) if bias.dim() == 1 else gx


def bias_gelu(x, bias):
    return _BiasGelu.apply(x, bias)


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


def _segments(cu_seqlens, T):
    if cu_seqlens is None:
        return [(0, T)]
    cs = cu_seqlens.tolist()
    return list(zip(cs[:-1], cs[1:]))


def attention_varlen(q, k, v, cu_seqlens=None, causal=True, scale=None, alibi_slopes=None, dropout_p=0.0):
    """Exact attention over packed documents.  q ``[T,Hq,D]``, k/v ``[T,Hk,D]`` (GQA when
    Hk < Hq: query head h reads kv head ``h // (Hq/Hk)``).  fp32 softmax; ``dropout_p`` drops attention
    probabilities (training only: the caller passes 0 in eval mode)."""
    T, Hq, D = q.shape
    Hk = k.shape[1]
    rep = Hq // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty_like(q)
    for a, b in _segments(cu_seqlens, T):
        if b <= a:
            continue
        qs = q[a:b].transpose(0, 1).float()
        ks = k[a:b].transpose(0, 1).float()
        vs = v[a:b].transpose(0, 1).float()
        if rep > 1:
            ks = ks.repeat_interleave(rep, dim=0)
            vs = vs.repeat_interleave(rep, dim=0)
        s = torch.matmul(qs, ks.transpose(1, 2)) * scale
        n = b - a
        if alibi_slopes is not None:
            pos = torch.arange(n, device=q.device)
            s = s + alibi_slopes.float().view(-1, 1, 1) * (pos.view(1, 1, n) - pos.view(1, n, 1))
        if causal:
            m = torch.ones(n, n, dtype=torch.bool, device=q.device).tril_()
            s = s.masked_fill(~m, float("-inf"))
        p = torch.softmax(s, dim=-1)
        if dropout_p:
            p = torch.nn.functional.dropout(p, dropout_p)
        out[a:b] = torch.matmul(p, vs).transpose(0, 1).to(q.dtype)
    return out


def attention_kvcache(q, k_cache, v_cache, q_pos0, scale=None):
    """Decode/prefill attention against a KV cache.  q ``[B,Sq,Hq,D]``; caches ``[B,Sk,Hk,D]``
    (already containing this step's keys); query i sits at absolute position ``q_pos0+i``."""
    B, Sq, Hq, D = q.shape
    Sk, Hk = k_cache.shape[1], k_cache.shape[2]
    rep = Hq // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qs = q.permute(0, 2, 1, 3).float()
    ks = k_cache.permute(0, 2, 1, 3).float().repeat_interleave(rep, dim=1)
    vs = v_cache.permute(0, 2, 1, 3).float().repeat_interleave(rep, dim=1)
    s = torch.matmul(qs, ks.transpose(-1, -2)) * scale
    qi = torch.arange(Sq, device=q.device).view(Sq, 1) + q_pos0
    kj = torch.arange(Sk, device=q.device).view(1, Sk)
    s = s.masked_fill(kj > qi, float("-inf"))
    return torch.matmul(torch.softmax(s, -1), vs).permute(0, 2, 1, 3).to(q.dtype)


def cross_entropy_parts(logits, target, vocab_start, valid_cols):
    """Per-token partial statistics of a vocab shard: (row max, sum exp(l - max), target logit
    or 0 when the target lives on another shard).  ``valid_cols`` excludes a padded tail."""
    lf = logits.float()[:, :valid_cols]
    mx = lf.max(dim=-1).values
    se = torch.exp(lf - mx.unsqueeze(-1)).sum(-1)
    local = target - vocab_start
    hit = (local >= 0) & (local < valid_cols)
    idx = torch.where(hit, local, torch.zeros_like(local))
    tl = torch.where(hit, lf.gather(1, idx.unsqueeze(1)).squeeze(1), torch.zeros_like(mx))
    return mx, se, tl


def adam_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, adamw=True, grad_scale=1.0,
              bias_correction=True):
    """One fp32 Adam(W) update in place on (p, m, v); ``g`` is multiplied by ``grad_scale``
    first (un-scale / clip coefficient folded in)."""
    g = g.float() * grad_scale
    if not adamw and weight_decay:
        g = g + weight_decay * p
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    if bias_correction:
        c1 = 1 - beta1 ** step
        c2 = 1 - beta2 ** step
    else:
        c1 = c2 = 1.0
    denom = (v / c2).sqrt_().add_(eps)
    upd = (m / c1) / denom
    if adamw and weight_decay:
        upd = upd + weight_decay * p
    p.add_(upd, alpha=-lr)
