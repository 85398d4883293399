"""Megatron-DeepSpeed *layer-file* checkpoints.

On-disk layout (the contract the reference's converter and loaders read —
tools/convert_ds_weight_to_hf_fast.py:205-246, llm/models/mg_models/llama/utils.py:353-439):

    <save_dir>/latest                                             text file holding the tag
    <save_dir>/<tag>/layer_{idx:02d}-model_{tp:02d}-model_states.pt   one per parameter-bearing
                                                                  layer and TP rank; idx = position
                                                                  in the spec list (1 embed,
                                                                  3…L+2 blocks, L+4 norm, L+5 head)
    <save_dir>/<tag>/mp_rank_{tp:02d}_model_states.pt             client state, lr scheduler, counters
    <save_dir>/<tag>/[bf16_]zero_pp_rank_{dp}_mp_rank_{mp:02d}_optim_states.pt   optimizer shard
                                                                  (mp = pp_rank·TP + tp_rank)

Layer files are sharded by TP only, so a checkpoint can be resumed under a different PP / DP
layout: stages load the layer indices they own, and optimizer shards are re-assembled by
parameter name when the DP size changed (``ZeroOptimizer.load_resharded``).
Files are written to ``<name>.tmp`` and renamed, so a crash never leaves a truncated file
under a final name; ``latest`` is updated last.
"""
from __future__ import annotations

import glob
import os
import re

import torch
import torch.distributed as dist

from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger

LAYER_RE = re.compile(r"layer_(\d+)-model_(\d+)-model_states\.pt$")


def layer_file(ckpt_dir, idx, tp_rank):
    return os.path.join(ckpt_dir, f"layer_{idx:02d}-model_{tp_rank:02d}-model_states.pt")


def mp_state_file(ckpt_dir, tp_rank):
    return os.path.join(ckpt_dir, f"mp_rank_{tp_rank:02d}_model_states.pt")


def zero_file(ckpt_dir, dp_rank, mp_rank, bf16=True):
    return os.path.join(ckpt_dir, f"{'bf16_' if bf16 else ''}zero_pp_rank_{dp_rank}_mp_rank_{mp_rank:02d}_optim_states.pt")


def atomic_save(obj, path):
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def safe_load(path, map_location="cpu"):
    try:
        return torch.load(path, map_location=map_location, weights_only=False)
    except Exception as e:  # truncated / corrupt file: name it instead of a bare unpickling error
        raise RuntimeError(f"checkpoint file {path} is unreadable ({type(e).__name__}: {e})") from e


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def read_latest(load_dir):
    p = os.path.join(load_dir, "latest")
    if not os.path.exists(p):
        return None
    with open(p) as f:
        return f.read().strip()


def save_layer_states(model, ckpt_dir, only=None):
    """Write this stage's layer files (caller restricts to dp_rank 0).  ``only`` filters keys."""
    g = get_grid()
    for key, mod in model.layers.items():
        sd = {k: v.detach().cpu().clone() for k, v in mod.state_dict().items()}
        if only is not None:
            sd = {k: v for k, v in sd.items() if only(int(key), k)}
            if not sd:
                continue
        atomic_save(sd, layer_file(ckpt_dir, int(key), g.tp_rank))


def load_layer_states(model, ckpt_dir, strict=True):
    g = get_grid()
    for key, mod in model.layers.items():
        path = layer_file(ckpt_dir, int(key), g.tp_rank)
        if not os.path.exists(path):
            if strict:
                raise FileNotFoundError(path)
            continue
        sd = safe_load(path)
        sd = {k: v for k, v in sd.items() if not k.endswith("rotary_emb.inv_freq")}
        missing, unexpected = mod.load_state_dict(sd, strict=False)
        missing = [m for m in missing if "lora_" not in m]
        if strict and (missing or unexpected):
            raise RuntimeError(f"{path}: missing {missing}, unexpected {unexpected}")


def save_engine_checkpoint(engine, save_dir, tag, client_state, save_base_state=True, save_zero=True,
                           save_optim=True):
    g = get_grid()
    tag = tag or f"global_step{engine.global_steps}"
    ckpt_dir = os.path.join(save_dir, str(tag))
    if g.rank == 0:
        os.makedirs(ckpt_dir, exist_ok=True)
    _barrier()
    os.makedirs(ckpt_dir, exist_ok=True)
    if g.dp_rank == 0:
        save_layer_states(engine.module, ckpt_dir)
        if g.pp_rank == 0:
            state = {"global_steps": engine.global_steps, "global_samples": engine.global_samples,
                     "skipped_steps": engine.skipped_steps, "dp_world_size": g.dp, "mp_world_size": g.tp,
                     "pp_world_size": g.pp,
                     "lr_scheduler": engine.lr_scheduler.state_dict() if engine.lr_scheduler is not None else None,
                     "ds_config": engine.config, "module": None}
            state.update(client_state)
            if not save_base_state:
                for k in ("iteration", "samples", "tokens"):
                    state.pop(k, None)
            atomic_save(state, mp_state_file(ckpt_dir, g.tp_rank))
    if save_optim and save_zero and engine.optimizer is not None and hasattr(engine.optimizer, "state_dict"):
        opt = engine.optimizer
        stage = getattr(opt, "stage", 0)
        if stage >= 1 or g.dp_rank == 0:
            sd = {"optimizer_state_dict": opt.state_dict(), "ds_version": "easyllm_b200"}
            atomic_save(sd, zero_file(ckpt_dir, g.dp_rank, g.pp_rank * g.tp + g.tp_rank, bf16=engine.bfloat16_enabled()))
    _barrier()
    if g.rank == 0:
        with open(os.path.join(save_dir, "latest.tmp"), "w") as f:
            f.write(str(tag))
        os.replace(os.path.join(save_dir, "latest.tmp"), os.path.join(save_dir, "latest"))
    _barrier()
    return True


def load_engine_checkpoint(engine, load_dir, tag=None, load_optimizer_states=True, load_zero=True,
                           load_lr_scheduler_states=True):
    g = get_grid()
    tag = tag or read_latest(load_dir)
    if tag is None:
        logger.warning(f"no 'latest' file in {load_dir}; nothing loaded")
        return None, {}
    ckpt_dir = os.path.join(load_dir, str(tag))
    load_layer_states(engine.module, ckpt_dir)
    state = safe_load(mp_state_file(ckpt_dir, g.tp_rank))
    engine.global_steps = state.get("global_steps", 0)
    engine.global_samples = state.get("global_samples", 0)
    engine.skipped_steps = state.get("skipped_steps", 0)
    if load_lr_scheduler_states and engine.lr_scheduler is not None and state.get("lr_scheduler") is not None:
        engine.lr_scheduler.load_state_dict(state["lr_scheduler"])
    opt = engine.optimizer
    if opt is not None and hasattr(opt, "refresh_fp32_params"):
        opt.refresh_fp32_params()
    if opt is not None and load_optimizer_states and load_zero and hasattr(opt, "load_resharded"):
        mp = g.pp_rank * g.tp + g.tp_rank
        bf16 = engine.bfloat16_enabled()
        mine = zero_file(ckpt_dir, g.dp_rank if getattr(opt, "stage", 0) >= 1 else 0, mp, bf16)
        same_layout = state.get("dp_world_size") == g.dp and state.get("pp_world_size", g.pp) == g.pp
        if same_layout and os.path.exists(mine):
            opt.load_state_dict(safe_load(mine)["optimizer_state_dict"])
        else:
            pat = zero_file(ckpt_dir, 0, mp, bf16).replace("pp_rank_0_", "pp_rank_*_")
            shards = [safe_load(p)["optimizer_state_dict"] for p in sorted(glob.glob(pat))]
            if shards and state.get("pp_world_size", g.pp) == g.pp:
                opt.load_resharded(shards)
            else:
                logger.warning("optimizer shards not found or pipeline layout changed: optimizer state starts fresh")
    elif opt is not None and load_optimizer_states and load_zero and hasattr(opt, "load_state_dict"):
        # optimizers driven through the adapter (SophiaG, Adam8bit, NovoGrad, SGD, torch.optim.*): replicated over
        # DP, saved once by the first DP rank
        path = zero_file(ckpt_dir, 0, g.pp_rank * g.tp + g.tp_rank, engine.bfloat16_enabled())
        if os.path.exists(path):
            opt.load_state_dict(safe_load(path)["optimizer_state_dict"])
        else:
            logger.warning(f"no optimizer state at {path}: the optimizer starts with fresh moments and step count")
    client = {k: v for k, v in state.items() if k not in ("lr_scheduler", "ds_config", "module")}
    _barrier()
    return ckpt_dir, client
