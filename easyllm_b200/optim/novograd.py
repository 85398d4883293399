"""NovoGrad: Adam-like update whose second moment is ONE scalar per tensor (the running squared gradient norm).

The reference's optimizer builder offers apex ``FusedNovoGrad`` (llm/utils/model/optimizer_helper.py:70-98); this is
the same update rule in PyTorch for the single-axis runners, with apex's defaults and options:

    v_t = ‖g‖²                                  first step, unless ``init_zero``
    v_t = β2·v + (1−β2)·‖g‖²                    afterwards (``norm_type=2``; ``norm_type=0`` uses max|g|)
    u   = g / (sqrt(v_t / c2) + eps)            c2 = 1−β2^t with ``bias_correction`` else 1
    u  += weight_decay · w                      (``reg_inside_moment=False``: added after the normalisation)
    m_t = β1·m + (1−β1 if grad_averaging else 1)·u
    w  -= lr · m_t / c1                         c1 = 1−β1^t with ``bias_correction`` else 1
"""
from __future__ import annotations

import torch
from torch.optim.optimizer import Optimizer


class NovoGrad(Optimizer):
    def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 amsgrad=False, reg_inside_moment=False, grad_averaging=True, norm_type=2, init_zero=False,
                 set_grad_none=True):
        if amsgrad:
            raise RuntimeError("NovoGrad does not support the AMSGrad variant")
        if norm_type not in (0, 2):
            raise RuntimeError("NovoGrad only supports the l2 (2) and infinity (0) norms")
        if lr < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("invalid NovoGrad hyper-parameters")
        super().__init__(params, dict(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                                      weight_decay=weight_decay, grad_averaging=grad_averaging, norm_type=norm_type,
                                      init_zero=init_zero, reg_inside_moment=reg_inside_moment))
        self.set_grad_none = set_grad_none

    def zero_grad(self, set_to_none=None):
        super().zero_grad(set_to_none=self.set_grad_none if set_to_none is None else set_to_none)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            t = group["step"]
            c1 = 1 - b1 ** t if group["bias_correction"] else 1.0
            c2 = 1 - b2 ** t if group["bias_correction"] else 1.0
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("NovoGrad does not support sparse gradients")
                g = p.grad.float()
                st = self.state[p]
                gn = g.abs().max() if group["norm_type"] == 0 else g.pow(2).sum()
                if "exp_avg" not in st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["v"] = torch.zeros((), dtype=torch.float32, device=p.device) if group["init_zero"] else gn.clone()
                    if group["init_zero"]:
                        st["v"].mul_(b2).add_(gn, alpha=1 - b2)
                elif group["norm_type"] == 0:
                    st["v"] = torch.maximum(st["v"] * b2, gn)
                else:
                    st["v"].mul_(b2).add_(gn, alpha=1 - b2)
                denom = (st["v"] / c2).sqrt() if group["norm_type"] == 2 else st["v"] / c2
                w = p.float()
                if group["reg_inside_moment"] and group["weight_decay"]:
                    g = g + group["weight_decay"] * w
                u = g / (denom + group["eps"])
                if not group["reg_inside_moment"] and group["weight_decay"]:
                    u = u + group["weight_decay"] * w
                st["exp_avg"].mul_(b1).add_(u, alpha=(1 - b1) if group["grad_averaging"] else 1.0)
                p.add_((-group["lr"] / c1 * st["exp_avg"]).to(p.dtype))
        return loss
