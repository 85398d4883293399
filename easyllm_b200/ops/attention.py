"""Dispatch to the sm_100a flash-attention kernels (``csrc/flash_attn.cu``)."""
from __future__ import annotations

import torch


def supported(q, k, v):
    from . import cuda
    return cuda.has_symbol("ell_flash_attn_fwd") and q.dtype == torch.bfloat16 and q.shape[-1] == 128


def flash_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale):
    from . import cuda
    return cuda.flash_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale)
