"""Engine contract of ``ZeroOptimizer`` over any ``torch.optim.Optimizer``.

The engines (``PipelineEngine``, ``ZeroDPEngine``), the checkpoint code and the logger hooks talk to the optimizer
through a small surface: ``accumulate_grads``, ``step`` (reduce → clip → update → zero; returns False when skipped),
``cur_scale``, ``get_global_grad_norm``, ``param_groups``, ``state_dict`` / ``load_state_dict``, ``zero_grad``,
``refresh_fp32_params``.  ``TorchOptimizerAdapter`` provides it for the optimizers that are not the native fused
Adam — SophiaG, NovoGrad, Adam8bit, SGD, any ``torch.optim`` class named in ``trainer.optimizer.type``
(llm/utils/model/optimizer_helper.py:70-98) — with plain data parallelism (ZeRO stage 0):

* every parameter gets an fp32 ``main_grad`` that micro-batch gradients are added into (the wgrad kernels of the
  native path write there directly; autograd ``.grad`` tensors are folded in by ``accumulate_grads``);
* ``step`` averages ``main_grad`` over the DP group, sums the gradients of TP-replicated sequence-parallel
  parameters over the TP group, clips by the global norm (replicated parameters counted once), hands the result to
  the wrapped optimizer as ``.grad`` and clears the accumulators.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel.grid import get_grid


class TorchOptimizerAdapter:
    stage = 0

    def __init__(self, optimizer: torch.optim.Optimizer, named_params, grad_clip=0.0, nan_policy="count"):
        self.inner = optimizer
        self.grid = get_grid()
        self.grad_clip, self.nan_policy = grad_clip, nan_policy
        self.names, self.params = [], []
        for n, p in named_params:
            if p.requires_grad:
                self.names.append(n)
                self.params.append(p)
                p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        self.skipped_steps = 0
        self.step_count = 0
        self._norm = None

    # ---- surface shared with ZeroOptimizer ------------------------------------------------------------------
    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def cur_scale(self):
        return 1.0

    def get_global_grad_norm(self):
        return None if self._norm is None else float(self._norm)

    def refresh_fp32_params(self):
        pass                                               # the wrapped optimizer updates the parameters in place

    def zero_grad(self):
        for p in self.params:
            p.main_grad.zero_()
            p.grad = None

    def accumulate_grads(self):
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    def _reduce(self):
        g = self.grid
        for p in self.params:
            if g.tp > 1 and (getattr(p, "sequence_parallel", False) or getattr(p, "tp_reduce_grad", False)):
                dist.all_reduce(p.main_grad, group=g.tp_group)
            if g.dp > 1:
                p.main_grad.div_(g.dp)
                dist.all_reduce(p.main_grad, group=g.dp_group)

    def _global_norm(self):
        g = self.grid
        sq = torch.zeros((), dtype=torch.float32, device=self.params[0].device)
        for p in self.params:
            replicated = not getattr(p, "tensor_model_parallel", False)
            if replicated and g.tp_rank != 0:
                continue                                   # count TP-replicated parameters once
            sq = sq + p.main_grad.pow(2).sum()
        if dist.is_initialized() and g.mp_group is not None and g.tp * g.pp > 1:
            dist.all_reduce(sq, group=g.mp_group)
        return sq.sqrt()

    def step(self, **kw):
        self._reduce()
        norm = self._global_norm()
        self._norm = norm
        if self.nan_policy in ("skip", "abort") and not bool(torch.isfinite(norm)):
            if self.nan_policy == "abort":
                raise FloatingPointError("non-finite gradient norm")
            self.skipped_steps += 1
            self.zero_grad()
            return False
        coef = 1.0
        if self.grad_clip and self.grad_clip > 0:
            coef = min(1.0, float(self.grad_clip / (norm + 1e-6)))
        for p in self.params:
            p.grad = (p.main_grad * coef).to(p.dtype)
        self.inner.step(**kw)
        self.step_count += 1
        self.zero_grad()
        return True

    # ---- checkpoint -------------------------------------------------------------------------------------------
    def state_dict(self):
        return {"inner": self.inner.state_dict(), "step": self.step_count, "skipped_steps": self.skipped_steps,
                "names": self.names, "kind": type(self.inner).__name__}

    def load_state_dict(self, sd, **_):
        self.inner.load_state_dict(sd["inner"])
        self.step_count, self.skipped_steps = sd.get("step", 0), sd.get("skipped_steps", 0)
