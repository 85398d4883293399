"""Optimizer construction from the ``trainer.optimizer`` config block.

Parity: llm/utils/model/optimizer_helper.py:19-98.  ``FusedAdam`` / ``AdamW`` / ``Adam`` map
to the native fused Adam on ZeRO-sharded flat buffers (decay / no-decay split: biases and
1-D parameters are not decayed; frozen parameters are left out).  ``FusedSGD`` maps to
``torch.optim.SGD``, ``FusedNovoGrad`` to ``optim.novograd.NovoGrad``; ``SophiaG`` and any
``torch.optim.*`` class are available for the single-axis runners; ``Adam8bit`` /
``AdamW8bit`` map to ``optim.adam8bit.Adam8bit`` (block-wise 8-bit optimizer state).
"""
from __future__ import annotations

import torch

from .zero import ZeroOptimizer

_NATIVE = {"FusedAdam": True, "AdamW": True, "Adam": False, "FusedAdamW": True}


def param_groups_weight_decay(model, weight_decay):
    decay, no_decay = [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (no_decay if (n.endswith(".bias") or p.dim() == 1) else decay).append(p)
    return [{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}]


def build_optimizer(cfg_optim, model, zero_stage=0, grad_clip=0.0, fp16=False, nan_policy="count",
                    engine_contract=False):
    """``engine_contract``: wrap optimizers other than the native fused Adam so that the training engines can drive
    them (accumulation into ``main_grad``, DP / TP gradient reduction, clipping); the runners pass True."""
    kind = cfg_optim["type"]
    kw = dict(cfg_optim.get("kwargs") or {})
    if kind in _NATIVE:
        adamw = kw.pop("adam_w_mode", _NATIVE[kind])
        return ZeroOptimizer(model.named_parameters(), lr=kw.get("lr", 1e-4), betas=tuple(kw.get("betas", (0.9, 0.999))),
                             eps=kw.get("eps", 1e-8), weight_decay=kw.get("weight_decay", 0.0), adamw=adamw,
                             stage=zero_stage, grad_clip=grad_clip, fp16=fp16,
                             bias_correction=kw.get("bias_correction", True), nan_policy=nan_policy)
    groups = param_groups_weight_decay(model, kw.pop("weight_decay", 0.0))
    if kind in ("Adam8bit", "AdamW8bit"):
        from .adam8bit import Adam8bit
        inner = Adam8bit(groups, adamw=(kind == "AdamW8bit"), **kw)
    elif kind == "SophiaG":
        from .sophia import SophiaG
        inner = SophiaG(groups, **kw)
    elif kind in ("FusedNovoGrad", "NovoGrad"):
        from .novograd import NovoGrad
        inner = NovoGrad(groups, **kw)
    elif kind == "FusedSGD":
        for extra in ("wd_after_momentum", "materialize_master_grads", "set_grad_none"):
            kw.pop(extra, None)
        inner = torch.optim.SGD(groups, **kw)
    elif hasattr(torch.optim, kind):
        inner = getattr(torch.optim, kind)(groups, **kw)
    else:
        raise KeyError(f"unknown optimizer type {kind}")
    if not engine_contract:
        return inner
    # the engines drive every optimizer through the ZeroOptimizer surface
    from .torch_adapter import TorchOptimizerAdapter
    return TorchOptimizerAdapter(inner, model.named_parameters(), grad_clip=grad_clip, nan_policy=nan_policy, fp16=fp16)
