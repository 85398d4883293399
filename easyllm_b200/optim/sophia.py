"""SophiaG optimizer (llm/utils/model/sophia.py:7-185).

Sign-momentum with per-coordinate clipping by a Hessian estimate ``h``:
``p ← p·(1 − lr·wd) − lr · clamp(m / max(ρ·bs·h, 1e-15), −1, 1)``.  ``update_hessian()``
refreshes ``h`` as an EMA of squared gradients; callers that never invoke it get the
reference's behaviour (``h = 0`` → pure clipped sign-momentum).
"""
from __future__ import annotations

import torch
from torch.optim.optimizer import Optimizer


class SophiaG(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=1e-1, maximize=False,
                 capturable=False):
        if lr < 0 or rho < 0 or weight_decay < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid SophiaG hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay, maximize=maximize,
                                      capturable=capturable))

    def _state(self, p):
        st = self.state[p]
        if not st:
            st["step"] = 0
            st["exp_avg"] = torch.zeros_like(p, memory_format=torch.preserve_format)
            st["hessian"] = torch.zeros_like(p, memory_format=torch.preserve_format)
        return st

    @torch.no_grad()
    def update_hessian(self):
        for group in self.param_groups:
            _, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self._state(p)
                st["hessian"].mul_(beta2).addcmul_(p.grad, p.grad, value=1 - beta2)

    @torch.no_grad()
    def step(self, closure=None, bs=5120):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, _ = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("SophiaG does not support sparse gradients")
                g = -p.grad if group["maximize"] else p.grad
                st = self._state(p)
                st["step"] += 1
                p.mul_(1 - group["lr"] * group["weight_decay"])
                st["exp_avg"].mul_(beta1).add_(g, alpha=1 - beta1)
                ratio = (st["exp_avg"].abs() / (group["rho"] * bs * st["hessian"] + 1e-15)).clamp_(max=1.0)
                p.addcmul_(st["exp_avg"].sign(), ratio, value=-group["lr"])
        return loss
