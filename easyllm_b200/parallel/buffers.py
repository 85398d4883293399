"""Grow-only named scratch tensors (llm/utils/env/dist_env/memory_buffer.py:21-39).

Used for gathered sequence-parallel activations so the ``[s, b, h]`` buffer is allocated
once, not once per layer.  Keys are (name, dtype, device).
"""
from __future__ import annotations

import math

import torch


class GlobalMemoryBuffer:
    def __init__(self):
        self._bufs = {}

    def get_tensor(self, shape, dtype, name, device=None):
        device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        need = math.prod(shape)
        key = (name, dtype, str(device))
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < need:
            buf = torch.empty(need, dtype=dtype, device=device, requires_grad=False)
            self._bufs[key] = buf
        return buf[:need].view(*shape)

    def clear(self):
        self._bufs.clear()


_BUF = GlobalMemoryBuffer()


def get_global_memory_buffer():
    return _BUF
