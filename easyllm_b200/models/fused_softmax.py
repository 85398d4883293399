"""Scale + mask + softmax of attention scores for the non-flash attention path.

Parity: llm/models/mg_models/base_modules/layers/fused_softmax.py:115-239 (``FusedScaleMaskSoftmax``): the reference
picks between three external CUDA kernels (causal upper-triangular, general mask, no mask; 16 < sk <= 4096) and a
PyTorch fallback.  On B200 the flash-attention kernels are the hot path for every training configuration, so this
wrapper keeps the reference's interface and semantics on one fused PyTorch expression (fp32 softmax when asked,
additive ``-10000`` style masking through ``mask_func``, causal masking for ``attn_mask_type='causal'``); it serves
the paths flash attention does not cover (ALiBi inference with a KV cache, CPU runs).
"""
from __future__ import annotations

import torch
import torch.nn as nn


def attention_mask_func(scores, mask):
    """Reference masking convention: positions where ``mask`` is True are filled with -10000."""
    return scores.masked_fill(mask, -10000.0)


class FusedScaleMaskSoftmax(nn.Module):
    def __init__(self, input_in_fp16=False, input_in_bf16=False, attn_mask_type="causal",
                 scaled_masked_softmax_fusion=True, mask_func=attention_mask_func, softmax_in_fp32=True, scale=None):
        super().__init__()
        if input_in_fp16 and input_in_bf16:
            raise ValueError("both fp16 and bf16 flags cannot be active at the same time.")
        if scale is not None and not softmax_in_fp32:
            raise ValueError("softmax should be in fp32 when scaled")
        self.input_in_float16 = input_in_fp16 or input_in_bf16
        self.attn_mask_type = attn_mask_type
        self.fusion = scaled_masked_softmax_fusion     # kept for config compatibility; one code path here
        self.mask_func, self.softmax_in_fp32, self.scale = mask_func, softmax_in_fp32, scale

    def forward(self, scores, mask=None):
        """scores ``[b, heads, sq, sk]``; ``mask`` broadcastable boolean (True = masked) or None."""
        assert scores.dim() == 4
        dtype = scores.dtype
        x = scores.float() if (self.input_in_float16 and self.softmax_in_fp32) else scores
        if self.scale is not None:
            x = x * self.scale
        if self.attn_mask_type == "causal":
            sq, sk = x.shape[-2:]
            causal = torch.ones(sq, sk, dtype=torch.bool, device=x.device).triu(diagonal=1 + sk - sq)
            x = x.masked_fill(causal, float("-inf"))
        if mask is not None:
            x = self.mask_func(x, mask)
        p = torch.softmax(x, dim=-1)
        return p.to(dtype) if p.dtype != dtype else p
