"""8-bit KV-cache quantisation for decoding (Qwen's ``use_cache_quantization``).

Parity: ``quantize_cache_v`` / ``dequantize_cache_torch`` of llm/models/hf_models/qwen/modeling_qwen.py:117-143 —
asymmetric uint8 quantisation of a chunk of keys or values with one (scale, zero) pair per (batch, head), taken over
all positions and channels of the chunk; ``x ≈ scale · (q − zero)``.  Chunks appended to a cache keep their own
pairs, stored per position so the cache can be sliced and concatenated along the sequence.

Layout here is the decode cache's ``[batch, seq, heads, head_dim]`` (the reference transposes to
``[batch, heads, seq, head_dim]`` first; the statistics are the same).
"""
from __future__ import annotations

import torch


def quantize_cache_v(fdata: torch.Tensor, bits: int = 8, qmax=None, qmin=None):
    """``fdata [b, s, h, d]`` → ``(uint8 [b, s, h, d], scale [b, s, h, 1], zero [b, s, h, 1])`` (fp32 pairs)."""
    qmax = float(2 ** bits - 1) if qmax is None else float(qmax)
    qmin = 0.0 if qmin is None else float(qmin)
    x = fdata.float()
    fmax = x.amax(dim=(1, 3), keepdim=True)
    fmin = x.amin(dim=(1, 3), keepdim=True)
    scale = ((fmax - fmin) / (qmax - qmin)).clamp_min(1e-12)       # a constant chunk must not divide by zero
    zero = qmin - fmin / scale
    q = torch.clamp(x / scale + zero, qmin, qmax).to(torch.uint8)
    shape = (x.shape[0], x.shape[1], x.shape[2], 1)
    return q.contiguous(), scale.expand(shape).contiguous(), zero.expand(shape).contiguous()


def dequantize_cache_torch(qdata: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, dtype=torch.float32):
    return (scale * (qdata.float() - zero)).to(dtype)


class QuantizedKV:
    """Pre-allocated uint8 cache for one layer: ``append`` quantises a chunk, ``read`` returns the dequantised
    prefix.  Holds 1 byte per element plus 8 bytes per (position, head) instead of 2 bytes per element."""

    def __init__(self, batch, max_len, heads, head_dim, device, dtype):
        self.q = torch.zeros(batch, max_len, heads, head_dim, dtype=torch.uint8, device=device)
        self.scale = torch.ones(batch, max_len, heads, 1, dtype=torch.float32, device=device)
        self.zero = torch.zeros(batch, max_len, heads, 1, dtype=torch.float32, device=device)
        self.dtype = dtype

    def append(self, p0, chunk):
        q, s, z = quantize_cache_v(chunk)
        n = chunk.shape[1]
        self.q[:, p0:p0 + n], self.scale[:, p0:p0 + n], self.zero[:, p0:p0 + n] = q, s, z

    def read(self, length):
        return dequantize_cache_torch(self.q[:, :length], self.scale[:, :length], self.zero[:, :length], self.dtype)
