"""LoRA for the HF-style models (the role peft plays in the reference:
llm/utils/general/hf_build_utils.py:20-27, tools/merge_base_model_with_lora.py:78-139).

``add_lora(model, cfg)`` freezes the base weights and attaches ``lora_A [r, in]`` /
``lora_B [out, r]`` to every ``nn.Linear`` whose attribute name is in ``target_modules``;
``adapter_state_dict`` / ``save_adapter`` use peft's key schema
(``base_model.model.<module>.lora_A.weight``) and ``merge_and_unload`` folds
``W += (alpha / r) · B · A`` back into the base weights.
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F


class LoraLinear(nn.Module):
    def __init__(self, base: nn.Linear, r, alpha, dropout):
        super().__init__()
        self.base = base
        self.r, self.scaling, self.dropout = r, alpha / r, dropout
        self.lora_A = nn.Parameter(torch.empty(r, base.in_features, dtype=base.weight.dtype, device=base.weight.device))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, r, dtype=base.weight.dtype, device=base.weight.device))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        for p in base.parameters():
            p.requires_grad = False

    @property
    def weight(self):            # fused-projection code concatenates .weight of q/k/v: give it the merged view
        return self.base.weight + self.scaling * (self.lora_B @ self.lora_A)

    @property
    def bias(self):
        return self.base.bias

    @property
    def in_features(self):
        return self.base.in_features

    @property
    def out_features(self):
        return self.base.out_features

    def forward(self, x):
        xd = F.dropout(x, self.dropout) if self.training and self.dropout > 0 else x
        return self.base(x) + F.linear(F.linear(xd, self.lora_A), self.lora_B) * self.scaling


def add_lora(model, cfg):
    targets = set(cfg.get("target_modules", ["q_proj", "v_proj"]))
    r, alpha, dropout = cfg.get("r", cfg.get("lora_rank", 8)), cfg.get("lora_alpha", 16), cfg.get("lora_dropout", 0.0)
    for p in model.parameters():
        p.requires_grad = False
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if name in targets and isinstance(child, nn.Linear):
                setattr(parent, name, LoraLinear(child, r, alpha, dropout))
    for name in cfg.get("modules_to_save") or []:
        for n, p in model.named_parameters():
            if name in n:
                p.requires_grad = True
    model.peft_config = dict(cfg, r=r, lora_alpha=alpha, lora_dropout=dropout, target_modules=sorted(targets))
    return model


def adapter_state_dict(model):
    out = {}
    for name, mod in model.named_modules():
        if isinstance(mod, LoraLinear):
            out[f"base_model.model.{name}.lora_A.weight"] = mod.lora_A.detach().cpu()
            out[f"base_model.model.{name}.lora_B.weight"] = mod.lora_B.detach().cpu()
    return out


def save_adapter(model, path):
    os.makedirs(path, exist_ok=True)
    torch.save(adapter_state_dict(model), os.path.join(path, "adapter_model.bin"))
    c = model.peft_config
    with open(os.path.join(path, "adapter_config.json"), "w") as f:
        json.dump({"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": c["r"], "lora_alpha": c["lora_alpha"],
                   "lora_dropout": c["lora_dropout"], "target_modules": c["target_modules"], "bias": "none"}, f, indent=2)


def load_adapter(model, path):
    """Wrap ``model`` with the LoRA layout recorded in ``path/adapter_config.json`` and load ``adapter_model.bin``
    (what ``PeftModel.from_pretrained`` does for the reference's ``peft_model_cfg.peft_path``)."""
    with open(os.path.join(path, "adapter_config.json")) as f:
        cfg = json.load(f)
    add_lora(model, {"r": cfg["r"], "lora_alpha": cfg["lora_alpha"], "lora_dropout": cfg.get("lora_dropout", 0.0),
                     "target_modules": cfg["target_modules"], "modules_to_save": cfg.get("modules_to_save")})
    sd = torch.load(os.path.join(path, "adapter_model.bin"), map_location="cpu")
    mods = dict(model.named_modules())
    loaded = 0
    for key, val in sd.items():
        name = key[len("base_model.model."):] if key.startswith("base_model.model.") else key
        for suffix, attr in ((".lora_A.weight", "lora_A"), (".lora_B.weight", "lora_B")):
            if name.endswith(suffix):
                mod = mods.get(name[:-len(suffix)])
                if not isinstance(mod, LoraLinear):
                    raise KeyError(f"{path}: adapter tensor {key} has no LoRA layer in the model")
                getattr(mod, attr).data.copy_(val.to(getattr(mod, attr)))
                loaded += 1
    expected = 2 * sum(isinstance(m, LoraLinear) for m in mods.values())
    if loaded != expected:
        raise KeyError(f"{path}: loaded {loaded} adapter tensors, the model has {expected}")
    return model


def merge_and_unload(model):
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if isinstance(child, LoraLinear):
                with torch.no_grad():
                    child.base.weight.add_((child.scaling * (child.lora_B.float() @ child.lora_A.float())).to(child.base.weight.dtype))
                setattr(parent, name, child.base)
    return model
