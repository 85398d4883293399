"""Autograd mappings between tensor-parallel / sequence-parallel regions.

Parity: llm/utils/env/dist_env/dist_mappings.py:222-373 (seven mappings) and the padded
``data_gather`` over the data-parallel group (:165-219).  These are the *composition*
forms built from ``torch.distributed`` collectives.  They are what runs on CPU/gloo, what
the unfused A/B path uses on GPUs, and the oracle for the fused all-gather→GEMM and
GEMM→reduce-scatter kernels, which replace the (mapping, matmul) pairs on the hot path.

  copy_to_tp            fwd identity            bwd all-reduce
  reduce_from_tp        fwd all-reduce          bwd identity
  scatter_to_tp         fwd split last dim      bwd all-gather last dim
  gather_from_tp        fwd all-gather last dim bwd split last dim
  scatter_to_sp         fwd split first dim     bwd all-gather first dim
  gather_from_sp        fwd all-gather first    bwd reduce-scatter first (or split)
  reduce_scatter_to_sp  fwd reduce-scatter      bwd all-gather first dim
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .grid import get_grid


def _tp():
    g = get_grid()
    return g.tp_group, g.tp, g.tp_rank


def all_reduce_tp(x):
    grp, n, _ = _tp()
    if n == 1:
        return x
    dist.all_reduce(x, group=grp)
    return x


def split_last_dim(x):
    _, n, r = _tp()
    if n == 1:
        return x
    return x.chunk(n, dim=-1)[r].contiguous()


def split_first_dim(x):
    _, n, r = _tp()
    if n == 1:
        return x
    if x.shape[0] % n:
        raise ValueError(f"first dim {x.shape[0]} is not divisible by tensor-parallel size {n}")
    c = x.shape[0] // n
    return x[r * c:(r + 1) * c].contiguous()


def gather_last_dim(x):
    grp, n, _ = _tp()
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=grp)
    return torch.cat(parts, dim=-1).contiguous()


def gather_first_dim(x, out=None):
    grp, n, _ = _tp()
    if n == 1:
        return x
    shape = list(x.shape)
    shape[0] *= n
    if out is None:
        out = torch.empty(shape, dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=grp)
    return out


def reduce_scatter_first_dim(x):
    grp, n, _ = _tp()
    if n == 1:
        return x
    if x.shape[0] % n:
        raise ValueError(f"first dim {x.shape[0]} is not divisible by tensor-parallel size {n}")
    shape = list(x.shape)
    shape[0] //= n
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    if dist.get_backend(grp) == "gloo":
        # gloo has no reduce_scatter: all-reduce then keep the local rows
        tmp = x.contiguous().clone()
        dist.all_reduce(tmp, group=grp)
        r = get_grid().tp_rank
        out.copy_(tmp[r * shape[0]:(r + 1) * shape[0]])
    else:
        dist.reduce_scatter_tensor(out, x.contiguous(), group=grp)
    return out


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return all_reduce_tp(g.contiguous().clone())


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return all_reduce_tp(x.contiguous().clone())

    @staticmethod
    def backward(ctx, g):
        return g


class _ScatterLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return split_last_dim(x)

    @staticmethod
    def backward(ctx, g):
        return gather_last_dim(g)


class _GatherLast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return gather_last_dim(x)

    @staticmethod
    def backward(ctx, g):
        return split_last_dim(g)


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return split_first_dim(x)

    @staticmethod
    def backward(ctx, g):
        return gather_first_dim(g)


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, rs_in_backward):
        ctx.rs = rs_in_backward
        return gather_first_dim(x)

    @staticmethod
    def backward(ctx, g):
        return (reduce_scatter_first_dim(g) if ctx.rs else split_first_dim(g)), None


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return reduce_scatter_first_dim(x)

    @staticmethod
    def backward(ctx, g):
        return gather_first_dim(g)


def copy_to_tensor_model_parallel_region(x): return _Copy.apply(x)
def reduce_from_tensor_model_parallel_region(x): return _Reduce.apply(x)
def scatter_to_tensor_model_parallel_region(x): return _ScatterLast.apply(x)
def gather_from_tensor_model_parallel_region(x): return _GatherLast.apply(x)
def scatter_to_sequence_parallel_region(x): return _ScatterSeq.apply(x)
def gather_from_sequence_parallel_region(x, tensor_parallel_output_grad=True): return _GatherSeq.apply(x, tensor_parallel_output_grad)
def reduce_scatter_to_sequence_parallel_region(x): return _ReduceScatterSeq.apply(x)


def data_gather(x, dst=0, group=None, pad_value=0):
    """Gather variable-length first-dim tensors of the data-parallel group on ``dst``
    (group-local index).  Returns the list of unpadded tensors on dst, ``None`` elsewhere."""
    g = get_grid()
    group = group if group is not None else g.dp_group
    n = dist.get_world_size(group) if group is not None else 1
    if n == 1:
        return [x]
    ranks = g.dp_ranks if group is g.dp_group else list(range(n))
    me = dist.get_rank(group)
    ln = torch.tensor([x.shape[0]], dtype=torch.long, device=x.device)
    lens = [torch.zeros_like(ln) for _ in range(n)]
    dist.all_gather(lens, ln, group=group)
    mx = int(max(t.item() for t in lens))
    pad = x.new_full((mx,) + tuple(x.shape[1:]), pad_value)
    pad[:x.shape[0]] = x
    bufs = [torch.empty_like(pad) for _ in range(n)]
    dist.all_gather(bufs, pad, group=group)
    if me != dst:
        return None
    return [b[:int(l.item())] for b, l in zip(bufs, lens)]
