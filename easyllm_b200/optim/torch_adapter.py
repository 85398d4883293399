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

    def __init__(self, optimizer: torch.optim.Optimizer, named_params, grad_clip=0.0, nan_policy="count", fp16=False,
                 loss_scale_cfg=None):
        from .zero import DynamicLossScaler
        self.inner = optimizer
        self.grid = get_grid()
        self.grad_clip, self.nan_policy = grad_clip, nan_policy
        self.names, self.params = [], []
        for n, p in named_params:
            if p.requires_grad:
                self.names.append(n)
                self.params.append(p)
                p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        # fp32 master copies: the wrapped optimizer never sees a bf16 / fp16 parameter (at fine-tuning learning
        # rates most updates are below half a bf16 ulp and would be rounded away); it updates the masters and the
        # model parameters are refreshed from them after every step
        self.masters = {}
        for group in self.inner.param_groups:
            swapped = []
            for p in group["params"]:
                if p.dtype != torch.float32 and p.requires_grad:
                    m = p.detach().clone().float().requires_grad_(True)
                    self.masters[p] = m
                    swapped.append(m)
                else:
                    swapped.append(p)
            group["params"] = swapped
        self.scaler = DynamicLossScaler(**(loss_scale_cfg or {})) if fp16 else None
        self.skipped_steps = 0
        self.step_count = 0
        self._norm = None

    # ---- surface shared with ZeroOptimizer ------------------------------------------------------------------
    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def cur_scale(self):
        return self.scaler.cur_scale if self.scaler else 1.0

    def get_global_grad_norm(self):
        return None if self._norm is None else float(self._norm)

    def refresh_fp32_params(self):
        """Re-read the masters from the model parameters (after weights were loaded into the model)."""
        with torch.no_grad():
            for p, m in self.masters.items():
                m.copy_(p)

    def zero_grad(self):
        for p in self.params:
            p.main_grad.zero_()
            p.grad = None
        for m in self.masters.values():
            m.grad = None

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
        return sq.sqrt() / self.cur_scale

    def step(self, **kw):
        self._reduce()
        norm = self._global_norm()
        self._norm = norm
        if self.scaler is not None or self.nan_policy in ("skip", "abort"):
            ok = bool(torch.isfinite(norm))
            if not ok:
                if self.scaler is not None:
                    self.scaler.update(True)           # overflow: skip the step, lower the scale
                elif self.nan_policy == "abort":
                    raise FloatingPointError("non-finite gradient norm")
                self.skipped_steps += 1
                self.zero_grad()
                return False
        coef = 1.0 / self.cur_scale
        if self.grad_clip and self.grad_clip > 0:
            coef *= min(1.0, float(self.grad_clip / (norm + 1e-6)))
        for p in self.params:
            m = self.masters.get(p)
            if m is not None:
                m.grad = p.main_grad * coef            # fp32 all the way
            else:
                p.grad = (p.main_grad * coef).to(p.dtype)
        self.inner.step(**kw)
        with torch.no_grad():
            for p, m in self.masters.items():
                p.copy_(m)
        if self.scaler is not None:
            self.scaler.update(False)
        self.step_count += 1
        self.zero_grad()
        return True

    # ---- checkpoint -------------------------------------------------------------------------------------------
    def state_dict(self):
        return {"inner": self.inner.state_dict(), "step": self.step_count, "skipped_steps": self.skipped_steps,
                "names": self.names, "kind": type(self.inner).__name__,
                "masters": [self.masters[p].detach().cpu() if p in self.masters else None for p in self.params],
                "scaler": self.scaler.state_dict() if self.scaler else None}

    def load_state_dict(self, sd, **_):
        if sd.get("kind") not in (None, type(self.inner).__name__):
            raise ValueError(f"checkpoint holds {sd.get('kind')} state, the run builds {type(self.inner).__name__}")
        if list(sd.get("names", self.names)) != list(self.names):
            raise ValueError("optimizer state was saved for a different set of trainable parameters "
                             f"({len(sd.get('names', []))} saved, {len(self.names)} now)")
        self.inner.load_state_dict(sd["inner"])
        self.step_count, self.skipped_steps = sd.get("step", 0), sd.get("skipped_steps", 0)
        saved = sd.get("masters")
        if saved is not None:
            with torch.no_grad():
                for p, m in zip(self.params, saved):
                    if m is not None and p in self.masters:
                        self.masters[p].copy_(m)
        if self.scaler and sd.get("scaler"):
            self.scaler.load_state_dict(sd["scaler"])
