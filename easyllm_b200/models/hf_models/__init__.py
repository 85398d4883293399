"""HF-runner model zoo: registry names of the reference → the generic ``CausalLM``.

``MODULE_ZOO_REGISTRY`` names kept: ``LlamaForCausalLM``, ``InternLMForCausalLM``,
``InternLM2ForCausalLM``, ``BaiChuanForCausalLM``, ``BaiChuan2ForCausalLM``,
``BaiChuan2ForCausalLM13B``, ``QWenForCausalLM``, ``QWenForVL``, ``KVLlamaForCausalLM``,
``medusa`` (llm/models/hf_models/*/__init__.py).  ``get_model_cfg`` mirrors
utils/model_utils.py:6-70: ``model_name_or_path``, ``torch_dtype``; the private
``_flash_*_2_enabled`` switches are accepted and ignored (the fused kernels are always on).
A config may give ``arch`` (a dict of HFArch fields) instead of a path to build a
random-initialised model of that shape.
"""
from __future__ import annotations

import torch

from ...config.registry import MODULE_ZOO_REGISTRY
from .modeling import CausalLM, HFArch, arch_from_hf_config, build_meta  # noqa: F401


def get_model_cfg(cfg):
    dt = cfg.get("torch_dtype", "torch.float32")
    if isinstance(dt, str):
        dt = getattr(torch, dt.replace("torch.", ""))
    return {"model_path": cfg.get("model_name_or_path"), "torch_dtype": dt}


def _builder(family):
    def build(**cfg):
        mc = get_model_cfg(cfg)
        if cfg.get("arch") is not None:
            arch = HFArch(family=family or "llama", **cfg["arch"])
            model = CausalLM(arch, mc["torch_dtype"])
        else:
            model = CausalLM.from_pretrained(mc["model_path"], family=family, torch_dtype=mc["torch_dtype"],
                                             arch_overrides=cfg.get("arch_overrides"))
        if cfg.get("model_parallel", False):
            model.is_parallelizable = True
            model.model_parallel = True
        return model
    return build


for _name, _fam in (("LlamaForCausalLM", "llama"), ("KVLlamaForCausalLM", "llama"), ("InternLMForCausalLM", "internlm"),
                    ("InternLM2ForCausalLM", "internlm2"), ("BaiChuanForCausalLM", "baichuan"),
                    ("BaiChuan2ForCausalLM", "baichuan2"), ("BaiChuan2ForCausalLM13B", "baichuan2-13b"),
                    ("QWenForCausalLM", "qwen")):
    MODULE_ZOO_REGISTRY.register(_name, _builder(_fam))

from . import medusa as _medusa  # noqa: E402,F401
from . import qwen_vl as _qwen_vl  # noqa: E402,F401
