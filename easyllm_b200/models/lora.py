"""Tensor-parallel LoRA adapters.

Parity: llm/models/mg_models/base_modules/lora/layers.py:15-228 and build_lora.py:5-64, plus
the trainable-parameter control and adapter checkpoint IO of llama/utils.py:353-582.

* column-parallel target (q/k/v/gate/up): ``A [r, in]`` replicated, ``B [out/tp, r]`` sharded;
* row-parallel target (o/down): ``A [r, in/tp]`` sharded, ``B [out, r]`` replicated, added to the
  partial output *before* the TP reduction so no extra collective is needed;
* vocab embedding / LM head: ``A [V/tp, r]`` (zeros) sharded, ``B [r, h]`` replicated.

Adapters attach to the existing (fused) layers — one adapter per named segment of the fused
q|k|v and gate|up projections — instead of swapping module classes; ``state_dict`` exposes the
reference's names (``self_attn.q_proj.lora_A_weight`` …).  Replicated halves are tagged
``tp_reduce_grad`` so their gradients are summed over the TP group once per step (the reference
averages the weights every forward instead).  Sequence parallelism is not supported with LoRA.
"""
from __future__ import annotations

import json
import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel import mappings as mp
from ..parallel.grid import get_grid
from ..parallel.rng import get_rng_tracker
from ..utils.log import default_logger as logger
from .layers import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding, _tag

COLUMN_TARGETS = ["gate_proj", "up_proj", "q_proj", "k_proj", "v_proj"]
ROW_TARGETS = ["down_proj", "o_proj"]
VOCAB_TARGETS = ["word_embeddings", "lm_head"]


class LoraPair(nn.Module):
    def __init__(self, a_shape, b_shape, a_sharded, b_sharded, dtype, device, a_init="kaiming", b_init="zeros"):
        super().__init__()
        self.lora_A_weight = nn.Parameter(torch.empty(*a_shape, dtype=dtype, device=device))
        self.lora_B_weight = nn.Parameter(torch.empty(*b_shape, dtype=dtype, device=device))
        for p, sharded, init, dim in ((self.lora_A_weight, a_sharded, a_init, 1), (self.lora_B_weight, b_sharded, b_init, 0)):
            _tag(p, sharded, dim if sharded else -1)
            if not sharded and get_grid().tp > 1:
                p.tp_reduce_grad = True
            ctx = get_rng_tracker().fork() if sharded and get_grid().tp > 1 else _null()
            with ctx:
                if init == "kaiming":
                    nn.init.kaiming_uniform_(p, a=math.sqrt(5))
                elif init == "normal":
                    nn.init.normal_(p)
                else:
                    nn.init.zeros_(p)


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _lora_cfg(cfg):
    return cfg["lora_rank"], cfg["lora_alpha"], cfg.get("lora_dropout", 0.0)


def _drop(x, p, training):
    return F.dropout(x, p) if training and p > 0 else x


def add_column_lora(mod: ColumnParallelLinear, segments, cfg):
    if mod.sequence_parallel:
        raise ValueError("Lora does not support sequence_parallel currently!")
    r, alpha, p = _lora_cfg(cfg)
    mod.lora = nn.ModuleDict()
    mod.lora_scaling, mod.lora_dropout = alpha / r, p
    dev, dt = mod.weight.device, mod.weight.dtype
    for (name, _), n_local in zip(mod.segments, mod.local_sizes):
        if name in segments or (name == "weight" and segments):
            mod.lora[name] = LoraPair((r, mod.in_features), (n_local, r), False, True, dt, dev)
    base_forward = mod.forward

    def forward(x):
        y = base_forward(x)
        if mod.gather_output:
            raise ValueError("LoRA on a gathering column-parallel linear is not supported")
        xin = mp.copy_to_tensor_model_parallel_region(x) if get_grid().tp > 1 else x
        xd = _drop(xin, mod.lora_dropout, mod.training)
        off = 0
        parts = []
        for (name, _), n_local in zip(mod.segments, mod.local_sizes):
            if name in mod.lora:
                pr = mod.lora[name]
                parts.append(F.linear(F.linear(xd, pr.lora_A_weight), pr.lora_B_weight) * mod.lora_scaling)
            else:
                parts.append(y.new_zeros(y.shape[0], n_local))
            off += n_local
        return y + torch.cat(parts, dim=-1)
    mod.forward = forward
    return mod


def add_row_lora(mod: RowParallelLinear, cfg):
    if mod.sequence_parallel:
        raise ValueError("Lora does not support sequence_parallel currently!")
    r, alpha, p = _lora_cfg(cfg)
    dev, dt = mod.weight.device, mod.weight.dtype
    pair = LoraPair((r, mod.in_local), (mod.out_features, r), True, False, dt, dev)
    mod.lora_A_weight, mod.lora_B_weight = pair.lora_A_weight, pair.lora_B_weight
    mod.lora_scaling, mod.lora_dropout = alpha / r, p

    def forward(x):
        from .. import ops
        if not mod.input_is_parallel:
            x = mp.scatter_to_tensor_model_parallel_region(x)
        y = ops.linear(x, mod.weight)
        y = y + F.linear(F.linear(_drop(x, mod.lora_dropout, mod.training), mod.lora_A_weight),
                         mod.lora_B_weight) * mod.lora_scaling
        if get_grid().tp > 1:
            y = mp.reduce_from_tensor_model_parallel_region(y)
        return y + mod.bias if mod.bias is not None else y
    mod.forward = forward
    return mod


def add_vocab_lora(mod: VocabParallelEmbedding, cfg):
    r, alpha, p = _lora_cfg(cfg)
    dev, dt = mod.weight.device, mod.weight.dtype
    pair = LoraPair((mod.per_rank, r), (r, mod.embedding_dim), True, False, dt, dev, a_init="zeros", b_init="normal")
    mod.lora_embedding_A_weight, mod.lora_embedding_B_weight = pair.lora_A_weight, pair.lora_B_weight
    mod.lora_embedding_A_weight.partition_dim = 0
    mod.lora_scaling = alpha / r
    base_lookup = mod.lookup

    def lookup(ids):
        out = base_lookup(ids)
        if get_grid().tp == 1:
            local, mask = ids, None
        else:
            mask = (ids < mod.vocab_start) | (ids >= mod.vocab_end)
            local = (ids - mod.vocab_start).masked_fill(mask, 0)
        extra = F.embedding(local, mod.lora_embedding_A_weight) @ mod.lora_embedding_B_weight * mod.lora_scaling
        if mask is not None:
            extra = extra.masked_fill(mask.unsqueeze(-1), 0.0)
        return out + extra
    mod.lookup = lookup
    return mod


def head_lora_logits(head, x):
    """LM-head LoRA (lm_head.py:10-46): logits += (x · Bᵀ?) — the embedding-shaped pair used as a
    linear map: ``x [T,h] · B_embᵀ [h,r] · A_embᵀ [r,V/tp]``."""
    emb = head.word_embeddings
    return (x @ emb.lora_embedding_B_weight.t()) @ emb.lora_embedding_A_weight.t() * emb.lora_scaling


def convert_layer_to_lora(model, cfg_lora):
    targets = list(cfg_lora.get("target_modules", []))
    for t in targets:
        if t not in COLUMN_TARGETS + ROW_TARGETS + VOCAB_TARGETS:
            raise ValueError(f"the module {t} is not support for lora now")
    L = model.num_layers
    for key, layer in model.layers.items():
        idx = int(key)
        if idx == 1 and "word_embeddings" in targets:
            add_vocab_lora(layer.word_embeddings, cfg_lora)
        elif idx == L + 5 and "lm_head" in targets:
            add_vocab_lora(layer.word_embeddings, cfg_lora)
            layer.lora_head = True
        elif hasattr(layer, "self_attn"):
            col_attn = [t for t in targets if t in ("q_proj", "k_proj", "v_proj")]
            col_mlp = [t for t in targets if t in ("gate_proj", "up_proj")]
            if col_attn:
                add_column_lora(layer.self_attn.qkv, col_attn, cfg_lora)
            if col_mlp:
                add_column_lora(layer.mlp.gate_up, col_mlp, cfg_lora)
            if "o_proj" in targets:
                add_row_lora(layer.self_attn.o_proj, cfg_lora)
            if "down_proj" in targets:
                add_row_lora(layer.mlp.down_proj, cfg_lora)
    model.lora_cfg = dict(cfg_lora)
    return model


def set_train_params(model, lora_mode=False, cfg_lora=None, is_train=True):
    """LoRA mode: only ``lora_*`` (and ``modules_to_save``: word_embeddings / lm_head) train."""
    if not (lora_mode and is_train):
        return
    L = model.num_layers
    save = ((cfg_lora or {}).get("saver") or {}).get("modules_to_save", [])
    for name, p in model.named_parameters():
        idx = int(name.split(".")[1])
        keep = "lora_" in name
        if idx == 1 and "word_embeddings" in save:
            keep = True
        if idx == L + 5 and "lm_head" in save:
            keep = True
        p.requires_grad = keep


def log_trainable_params(model):
    tot = sum(p.numel() for p in model.parameters())
    tr = sum(p.numel() for p in model.parameters() if p.requires_grad)
    g = get_grid()
    logger.info(f"stage {g.pp_rank}: trainable params {tr:,} / {tot:,} ({100.0 * tr / max(1, tot):.4f}%)")
    return tr, tot


# ---- adapter checkpoint IO ----------------------------------------------------------------------
def lora_state_filter(model, cfg_lora):
    L = model.num_layers
    save = ((cfg_lora or {}).get("saver") or {}).get("modules_to_save", [])

    def keep(idx, key):
        if "lora_" in key:
            return True
        return (idx == 1 and "word_embeddings" in save) or (idx == L + 5 and "lm_head" in save)
    return keep


def save_lora_ckpt_pretrained(cfg_lora, model, iteration=None):
    """``<save_path>[/iter_N]/layer_XX-model_YY-model_states.pt`` holding adapter tensors only, plus
    a peft-schema ``adapter_config.json``."""
    from ..ckpt.layer_files import save_layer_states
    g = get_grid()
    saver = cfg_lora["saver"]
    path = saver["save_path"]
    if iteration is not None and saver.get("save_by_iteration", True):
        path = os.path.join(path, f"global_step{iteration}")
    os.makedirs(path, exist_ok=True)
    if g.dp_rank == 0:
        save_layer_states(model, path, only=lora_state_filter(model, cfg_lora))
    if g.rank == 0:
        cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": cfg_lora["lora_rank"],
               "lora_alpha": cfg_lora["lora_alpha"], "lora_dropout": cfg_lora.get("lora_dropout", 0.0),
               "target_modules": [t if t != "word_embeddings" else "embed_tokens" for t in cfg_lora["target_modules"]],
               "base_model_name_or_path": cfg_lora.get("base_model_name_or_path"), "bias": "none",
               "fan_in_fan_out": False, "inference_mode": True, "init_lora_weights": True,
               "modules_to_save": saver.get("modules_to_save")}
        with open(os.path.join(path, "adapter_config.json"), "w") as f:
            json.dump(cfg, f, indent=2)
    return path


def _reshard(name, full, tp, rank):
    """This rank's slice of a merged (TP-free) adapter tensor, by the same rules that merge it."""
    from ..ckpt.ds_to_hf import LORA_COL, LORA_ROW
    if tp == 1:
        return full
    if LORA_COL.search(name):
        n = full.shape[0] // tp
        return full[rank * n:(rank + 1) * n].clone()
    if LORA_ROW.search(name):
        n = full.shape[1] // tp
        return full[:, rank * n:(rank + 1) * n].clone()
    return full                                            # replicated halves


def load_lora_from_ds_format(load_dir, model):
    """Adapter layer files written at any TP size: same size → this rank's files as they are; another size → the
    shards of every tensor are merged and re-cut for this rank (llm/models/mg_models/llama/utils.py:353-439)."""
    from ..ckpt.ds_to_hf import index_layer_files, merge_tensor
    from ..ckpt.layer_files import load_layer_states, safe_load
    g = get_grid()
    try:
        table, _ = index_layer_files(load_dir)
    except FileNotFoundError:
        return False
    saved_tp = max(len(v) for v in table.values())
    if saved_tp == g.tp:
        load_layer_states(model, load_dir, strict=False)
        return True
    for key, mod in model.layers.items():
        files = table.get(int(key))
        if not files:
            continue
        shards = [safe_load(files[r]) for r in sorted(files)]
        sd = {}
        for name in shards[0]:
            if "lora_" not in name:
                continue
            full = list(merge_tensor(name, [sh[name] for sh in shards]).values())[0]
            sd[name] = _reshard(name, full, g.tp, g.tp_rank)
        mod.load_state_dict(sd, strict=False)
    return True


def load_lora_from_hf_format(load_dir, model):
    """A peft adapter folder (``adapter_model.bin``, keys ``base_model.model.model.layers.N.….lora_A.weight``) into
    the TP-sharded adapter modules of this rank."""
    path = os.path.join(load_dir, "adapter_model.bin")
    if not os.path.exists(path):
        return False
    g = get_grid()
    sd = torch.load(path, map_location="cpu")
    per_layer = {}
    for k, v in sd.items():
        k = k.replace("base_model.model.", "", 1)
        if k.startswith("model.layers."):
            _, _, idx, rest = k.split(".", 3)
            lid, name = int(idx) + 3, rest.replace("lora_A.weight", "lora_A_weight").replace("lora_B.weight", "lora_B_weight")
        elif k.startswith("model.embed_tokens."):
            lid = 1
            name = "word_embeddings." + k.split(".", 2)[2].replace("lora_embedding_A", "lora_embedding_A_weight").replace(
                "lora_embedding_B", "lora_embedding_B_weight")
        elif k.startswith("lm_head."):
            lid = model.num_layers + 5
            name = "word_embeddings." + k.split(".", 1)[1].replace("lora_A.weight", "lora_embedding_A_weight").replace(
                "lora_B.weight", "lora_embedding_B_weight")
        else:
            continue
        per_layer.setdefault(lid, {})[name] = _reshard(name, v, g.tp, g.tp_rank)
    for key, mod in model.layers.items():
        if int(key) in per_layer:
            mod.load_state_dict(per_layer[int(key)], strict=False)
    return bool(per_layer)


def load_lora_ckpt_pretrained(cfg_lora, model, optimizer=None):
    loader = cfg_lora["loader"]
    if loader.get("debug", False):
        logger.info("skip loaded checkpoint for debug")
        return
    mode = loader.get("load_mode", "deepspeed")
    if mode == "deepspeed":
        ok = load_lora_from_ds_format(loader["load_path"], model)
    elif mode == "huggingface":
        ok = load_lora_from_hf_format(loader["load_path"], model)
    else:
        raise NotImplementedError(f"lora load mode {mode} is not support")
    if ok:
        logger.info(f"Successfully loaded lora checkpoint from {loader['load_path']}.")
        if optimizer is not None and hasattr(optimizer, "refresh_fp32_params"):
            optimizer.refresh_fp32_params()
    else:
        logger.info("Fail to load any lora checkpoints and will start from random.")


def merge_lora_into_hf_state(base_state, adapter_state, scaling):
    """W += scaling · B · A for every adapted HF linear / embedding; returns the merged dict."""
    out = dict(base_state)
    for k, a in adapter_state.items():
        if not k.endswith("lora_A.weight"):
            continue
        b = adapter_state[k.replace("lora_A.weight", "lora_B.weight")]
        target = k.replace("base_model.model.", "").replace(".lora_A.weight", ".weight")
        out[target] = (out[target].float() + scaling * (b.float() @ a.float())).to(out[target].dtype)
    for k, a in adapter_state.items():
        if k.endswith("lora_embedding_A"):
            b = adapter_state[k.replace("lora_embedding_A", "lora_embedding_B")]
            target = k.replace("base_model.model.", "").replace(".lora_embedding_A", ".weight")
            # layer-file convention: A [V, r], B [r, h]
            delta = a.float() @ b.float() if a.shape[0] == out[target].shape[0] else (b.float() @ a.float()).t()
            out[target] = (out[target].float() + scaling * delta).to(out[target].dtype)
    return out
