"""Every shipped YAML config loads, names registered components, and (Megatron set) expands into valid model arguments."""
import glob
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MEGATRON = sorted(glob.glob(os.path.join(ROOT, "configs", "megatron", "*.yaml")))
HF = sorted(glob.glob(os.path.join(ROOT, "configs", "huggingface", "*.yaml"))
            + glob.glob(os.path.join(ROOT, "configs", "huggingface", "inference", "*.yaml")))


def _registered(registry, cfg, what, path):
    if isinstance(cfg, dict) and "type" in cfg:
        assert cfg["type"] in registry, f"{path}: {what} type {cfg['type']!r} is not registered"


@pytest.mark.parametrize("path", MEGATRON, ids=[os.path.basename(p) for p in MEGATRON])
def test_megatron_config(path):
    from easyllm_b200.config import load_yaml
    from easyllm_b200.config.registry import (BATCH_CALCULATOR_REGISTRY, BATCH_COLLECTOR_REGISTRY, BATCH_FN_REGISTRY,
                                              BATCH_SAMPLER_REGISTRY, DATALOADER_REGISTRY, DATASET_REGISTRY,
                                              HOOK_REGISTRY, LR_REGISTRY, MODULE_ZOO_REGISTRY, TOKENIZER_REGISTRY)
    import easyllm_b200.data  # noqa: F401  (registers the data components)
    import easyllm_b200.models  # noqa: F401
    import easyllm_b200.optim  # noqa: F401
    import easyllm_b200.runners.hooks  # noqa: F401
    from easyllm_b200.models.config import LLAMA_PRESETS, update_model_cfg
    cfg = load_yaml(path)
    for key in ("runtime", "tokenizer", "data", "model"):
        assert key in cfg, (path, key)
    rt = cfg["runtime"]
    assert rt.get("tensor_model_parallel_size", 1) >= 1 and rt.get("pipeline_model_parallel_size", 1) >= 1
    _registered(TOKENIZER_REGISTRY, cfg["tokenizer"], "tokenizer", path)
    for split, d in cfg["data"].items():
        if not isinstance(d, dict):
            continue
        ds = d.get("dataset")
        for one in (ds if isinstance(ds, list) else [ds]):
            _registered(DATASET_REGISTRY, one, "dataset", path)
        _registered(BATCH_SAMPLER_REGISTRY, d.get("batch_sampler"), "batch_sampler", path)
        _registered(BATCH_COLLECTOR_REGISTRY, d.get("batch_collector"), "batch_collector", path)
        _registered(DATALOADER_REGISTRY, d.get("data_loader"), "data_loader", path)
        _registered(BATCH_FN_REGISTRY, d.get("batch_pipe"), "batch_pipe", path)
        _registered(BATCH_CALCULATOR_REGISTRY, d.get("batch_calculator"), "batch_calculator", path)
    if "trainer" in cfg:
        _registered(LR_REGISTRY, cfg["trainer"].get("lr_scheduler"), "lr_scheduler", path)
    for h in cfg.get("hooks") or []:
        _registered(HOOK_REGISTRY, h, "hook", path)
    model = cfg["model"]
    assert model["type"] in MODULE_ZOO_REGISTRY, (path, model["type"])
    kwargs = dict(LLAMA_PRESETS.get(model["type"], {}))
    kwargs.update(model.get("kwargs") or {})
    kwargs.setdefault("vocab_size", cfg["tokenizer"].get("pad_vocab_size_to") or 32000)
    args = update_model_cfg(kwargs)                      # raises on unknown keys / inconsistent sizes
    assert args.hidden_size % args.num_attention_heads == 0
    assert args.num_attention_heads % rt.get("tensor_model_parallel_size", 1) == 0


@pytest.mark.parametrize("path", HF, ids=[os.path.basename(p) for p in HF])
def test_huggingface_config(path):
    from easyllm_b200.config import load_yaml
    cfg = load_yaml(path)
    for key in ("runtime", "tokenizer", "data", "model", "trainer"):
        assert key in cfg, (path, key)
    assert "type" in cfg["model"]
