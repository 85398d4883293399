"""Broadcast of a micro-batch from tensor-parallel rank 0 to its TP group.

Parity: llm/utils/env/dist_env/dist_data.py:33-116 — only TP rank 0 owns a data loader; the
named int64 tensors of a micro-batch are flattened into one buffer and broadcast, preceded
by a fixed-size shape header.  Works on CPU (gloo) and GPU (NCCL) tensors.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .grid import get_grid

MAX_DIMS = 5


def _device():
    if torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def broadcast_data(keys, data, dtype=torch.int64):
    g = get_grid()
    if g.tp == 1:
        dev = _device()
        return {k: data[k].to(dev, non_blocking=True) for k in keys}
    dev = _device()
    src = g.tp_src_rank()
    header = torch.zeros(len(keys) * MAX_DIMS, dtype=torch.int64)
    if g.tp_rank == 0:
        for i, k in enumerate(keys):
            t = data[k]
            if t.dtype != dtype:
                raise TypeError(f"{k} has dtype {t.dtype}, expected {dtype}")
            if t.dim() >= MAX_DIMS:
                raise ValueError(f"{k}: rank {t.dim()} tensors need MAX_DIMS > {MAX_DIMS}")
            for j, s in enumerate(t.shape):
                header[i * MAX_DIMS + j] = s
    header = header.to(dev)
    dist.broadcast(header, src, group=g.tp_group)
    header = header.cpu().tolist()
    shapes, numels = {}, {}
    for i, k in enumerate(keys):
        dims = []
        for j in range(MAX_DIMS):
            s = header[i * MAX_DIMS + j]
            if s <= 0:
                break
            dims.append(s)
        shapes[k] = dims
        n = 1
        for s in dims:
            n *= s
        numels[k] = n
    total = sum(numels.values())
    if g.tp_rank == 0:
        flat = torch.cat([data[k].contiguous().view(-1) for k in keys]).to(dev)
    else:
        flat = torch.empty(total, dtype=dtype, device=dev)
    dist.broadcast(flat, src, group=g.tp_group)
    out, off = {}, 0
    for k in keys:
        out[k] = flat.narrow(0, off, numels[k]).view(shapes[k])
        off += numels[k]
    return out
