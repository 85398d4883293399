"""Precision boundary helpers of the pipeline model: cast what enters a half-precision model to its compute dtype
and what leaves it (logits, losses) back to fp32.

Parity: llm/models/mg_models/base_modules/modules/fp16_module.py:13-85 (``fp32_to_float16``, ``float16_to_fp32``,
``Float16Module``).  In this framework the parameters already live in the compute dtype inside the optimizer's flat
buffer (fp32 master copies are the optimizer's), so the wrapper only converts activations at the boundary.
"""
from __future__ import annotations

import torch
import torch.nn as nn

_HALF = (torch.float16, torch.bfloat16)


def _map(val, fn):
    if isinstance(val, (tuple, list)):
        out = [_map(v, fn) for v in val]
        return tuple(out) if isinstance(val, tuple) else out
    if isinstance(val, dict):
        return {k: _map(v, fn) for k, v in val.items()}
    return fn(val)


def fp32_to_float16(val, dtype=torch.bfloat16):
    """fp32 tensors (in arbitrarily nested tuples / lists / dicts) → ``dtype``; everything else untouched."""
    return _map(val, lambda t: t.to(dtype) if torch.is_tensor(t) and t.dtype == torch.float32 else t)


def float16_to_fp32(val):
    """fp16 / bf16 tensors (nested) → fp32; everything else untouched."""
    return _map(val, lambda t: t.float() if torch.is_tensor(t) and t.dtype in _HALF else t)


class Float16Module(nn.Module):
    """Runs ``module`` in half precision: parameters cast once, fp32 inputs cast on the way in, outputs on the way out."""

    def __init__(self, module, fp16=False, bf16=True):
        super().__init__()
        if fp16 == bf16:
            raise ValueError("choose exactly one of fp16 / bf16")
        self.dtype = torch.float16 if fp16 else torch.bfloat16
        self.module = module.to(self.dtype)

    def forward(self, *inputs, **kwargs):
        out = self.module(*fp32_to_float16(inputs, self.dtype), **fp32_to_float16(kwargs, self.dtype))
        return float16_to_fp32(out)

    def state_dict(self, *a, **k):
        return self.module.state_dict(*a, **k)

    def load_state_dict(self, sd, strict=True):
        return self.module.load_state_dict(sd, strict=strict)
