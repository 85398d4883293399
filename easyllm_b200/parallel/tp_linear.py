"""Tensor-parallel linear maps with Megatron-style sequence parallelism.

``column_parallel_linear``: the input is sequence-sharded ``[T/tp, K]`` (SP) or replicated
``[T, K]``; output ``[T, N/tp]``.  ``row_parallel_linear``: input ``[T, K/tp]``, output
reduce-scattered to ``[T/tp, N]`` (SP) or all-reduced ``[T, N]``.

Parity: llm/models/mg_models/base_modules/layers/column_parallel_linear.py:13-106 (forward
all-gather → GEMM; backward re-gather ‖ dgrad, reduce-scatter(dgrad) ‖ wgrad) and
row_parallel_linear.py:105-132.  Here one gather serves the fused q|k|v (or gate|up)
projection, so a layer gathers twice instead of five times.  These are the composition
forms (collective + GEMM as separate kernels, overlapped with async collectives); the fused
all-gather→GEMM / GEMM→reduce-scatter kernels register themselves through ``set_fused_impl``
and take over for CUDA bf16 inputs when a symmetric-memory workspace is installed.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from .buffers import get_global_memory_buffer
from .grid import get_grid
from . import mappings as mp

_FUSED = {"ag_gemm": None, "gemm_rs": None, "agk_wgrad": None}


def set_fused_impl(ag_gemm=None, gemm_rs=None, agk_wgrad=None):
    """Install fused kernels: ``ag_gemm(x_local, w, bias, b_mn=False, want_gathered=False) -> (y, x_gathered)``,
    ``gemm_rs(x, w, b_mn=False, all_reduce=False, push=None) -> y`` and ``agk_wgrad(dy, x_local, dw32,
    dry_run=False) -> True`` (each may return None for an unsupported shape; ``dry_run`` only asks).  ``None`` restores the composition."""
    _FUSED["ag_gemm"], _FUSED["gemm_rs"], _FUSED["agk_wgrad"] = ag_gemm, gemm_rs, agk_wgrad


def _use_fused(x):
    return x.is_cuda and x.dtype == torch.bfloat16 and ops.get_backend() == "b200"


def _ag_start(x, name):
    g = get_grid()
    shape = list(x.shape)
    shape[0] *= g.tp
    out = get_global_memory_buffer().get_tensor(shape, x.dtype, name, device=x.device)
    work = dist.all_gather_into_tensor(out, x.contiguous(), group=g.tp_group, async_op=True)
    return out, work


def _rs_start(x):
    g = get_grid()
    if dist.get_backend(g.tp_group) == "gloo":
        return mp.reduce_scatter_first_dim(x), None
    shape = list(x.shape)
    shape[0] //= g.tp
    out = torch.empty(shape, dtype=x.dtype, device=x.device)
    work = dist.reduce_scatter_tensor(out, x.contiguous(), group=g.tp_group, async_op=True)
    return out, work


def _wgrad(ctx_w, dy, x):
    """dW = dyᵀ·x delivered into main_grad (None returned) or as a tensor."""
    mg = getattr(ctx_w, "main_grad", None)
    if mg is not None:
        ops.matmul_tn_accum(dy, x, mg)
        return None
    return ops.matmul_tn(dy, x)


class _ColumnSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.wref, ctx.bref = w, bias
        fused = _FUSED["ag_gemm"] if _use_fused(x) else None
        res = fused(x, w, bias) if fused is not None else None
        if res is not None:
            y = res[0]
        else:
            xg, work = _ag_start(x, "sp_gather")
            work.wait()
            y = ops.matmul_nt(xg, w, bias)
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        fused_rs = _FUSED["gemm_rs"] if _use_fused(dy) else None
        fused_wg = _FUSED["agk_wgrad"] if _use_fused(dy) else None
        mg = getattr(ctx.wref, "main_grad", None)
        # weight gradient behind the re-gather of x in ONE kernel when it accumulates into the fp32 main_grad
        wg_fused = (fused_wg is not None and mg is not None and ctx.needs_input_grad[1]
                    and fused_wg(dy, x, mg, dry_run=True))
        ag_work = xg = None
        if ctx.needs_input_grad[1] and not wg_fused:
            xg, ag_work = _ag_start(x, "sp_gather_bwd")      # re-gather ‖ dgrad GEMM
        # the dgrad -> reduce-scatter launch also pushes x to the peers for the weight-gradient kernel behind it
        dx = (fused_rs(dy, w, b_mn=True, push=x if wg_fused else None)) if fused_rs is not None else None
        rs_work = None
        if dx is None:
            dxg = ops.matmul_nn(dy, w)
            dx, rs_work = _rs_start(dxg)                      # reduce-scatter ‖ wgrad GEMM
        dw = None
        if wg_fused and fused_wg(dy, x, mg) is None:
            xg, ag_work = _ag_start(x, "sp_gather_bwd")      # shape the fused kernel does not take
            wg_fused = False
        if ctx.needs_input_grad[1] and not wg_fused:
            ag_work.wait()
            dw = _wgrad(ctx.wref, dy, xg)
        db = None
        if ctx.bref is not None and ctx.needs_input_grad[2]:
            db = ops._grad_to(ctx.bref, ops.column_sum(dy))
        if rs_work is not None:
            rs_work.wait()
        return dx, dw, db


class _RowSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.wref = w
        ctx.save_for_backward(x, w)
        fused = _FUSED["gemm_rs"] if _use_fused(x) else None
        if fused is not None:
            out = fused(x, w)
            if out is not None:
                return out
        y = ops.matmul_nt(x, w)
        out, work = _rs_start(y)
        if work is not None:
            work.wait()
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        fused = _FUSED["ag_gemm"] if (_use_fused(dy) and ctx.needs_input_grad[0]) else None
        res = fused(dy, w, None, b_mn=True, want_gathered=ctx.needs_input_grad[1]) if fused is not None else None
        if res is not None:
            # dgrad as all-gather -> GEMM in one kernel; the gathered dy it leaves behind feeds the wgrad GEMM
            dx, dyg = res
            dw = _wgrad(ctx.wref, dyg, x) if ctx.needs_input_grad[1] else None
            return dx, dw
        dyg, work = _ag_start(dy, "sp_gather_row_bwd")
        work.wait()
        dx = ops.matmul_nn(dyg, w) if ctx.needs_input_grad[0] else None
        dw = _wgrad(ctx.wref, dyg, x) if ctx.needs_input_grad[1] else None
        return dx, dw


class _ColumnAR(torch.autograd.Function):
    """Column-parallel linear on a replicated input (no sequence parallelism): the forward needs no collective, the
    input gradient is the all-reduce of ``dy · W``, which the fused kernel produces in one launch
    (column_parallel_linear.py:68-86 of the reference: dgrad GEMM, then an all-reduce)."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.wref, ctx.bref = w, bias
        ctx.save_for_backward(x, w)
        return ops.matmul_nt(x, w, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            fused = _FUSED["gemm_rs"] if _use_fused(dy) else None
            dx = fused(dy, w, b_mn=True, all_reduce=True) if fused is not None else None
            if dx is None:
                dx = ops.matmul_nn(dy, w)
                dist.all_reduce(dx, group=get_grid().tp_group)
        dw = _wgrad(ctx.wref, dy, x) if ctx.needs_input_grad[1] else None
        db = None
        if ctx.bref is not None and ctx.needs_input_grad[2]:
            db = ops._grad_to(ctx.bref, ops.column_sum(dy))
        return dx, dw, db


class _RowAR(torch.autograd.Function):
    """Row-parallel linear whose output is all-reduced over TP (no sequence parallelism): GEMM and all-reduce
    in one kernel (row_parallel_linear.py:113-119 of the reference: F.linear, then ``_reduce``)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.wref = w
        ctx.save_for_backward(x, w)
        fused = _FUSED["gemm_rs"] if _use_fused(x) else None
        y = fused(x, w, all_reduce=True) if fused is not None else None
        if y is None:
            y = ops.matmul_nt(x, w)
            dist.all_reduce(y, group=get_grid().tp_group)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = ops.matmul_nn(dy, w) if ctx.needs_input_grad[0] else None
        dw = _wgrad(ctx.wref, dy, x) if ctx.needs_input_grad[1] else None
        return dx, dw


def _flat2(x):
    return x.reshape(-1, x.shape[-1]).contiguous()


def column_parallel_linear(x, w, bias=None, sequence_parallel=False):
    g = get_grid()
    if g.tp == 1:
        return ops.linear(x, w, bias)
    if sequence_parallel:
        return _ColumnSP.apply(x, w, bias)
    if _use_fused(x):
        return _ColumnAR.apply(_flat2(x), w, bias).view(*x.shape[:-1], w.shape[0])
    return ops.linear(mp.copy_to_tensor_model_parallel_region(x), w, bias)


def row_parallel_linear(x, w, bias=None, sequence_parallel=False):
    g = get_grid()
    if g.tp == 1:
        return ops.linear(x, w, bias)
    if sequence_parallel:
        y = _RowSP.apply(x, w)
    elif _use_fused(x):
        y = _RowAR.apply(_flat2(x), w).view(*x.shape[:-1], w.shape[0])
    else:
        y = mp.reduce_from_tensor_model_parallel_region(ops.linear(x, w))
    if bias is not None:
        y = y + bias
    return y
