"""Checkpoint policy of the runners (llm/utils/model/ckpt_helper.py:12-197).

``loader``: ``load_mode`` ``huggingface`` (HF weights → TP shards, ``pretrain_type`` llama /
llama_pack / internlm2 / internlm2_pack / qwen, ``debug`` skips the read) or ``deepspeed``
(layer-file checkpoint; ``load_optim`` / ``load_zero``; ``load_base_state`` restores iteration,
consumed samples and tokens; ``load_rng_state`` restores python / numpy / torch / device RNG and
the model-parallel RNG tracker).  ``saver``: ``save_mode`` ``deepspeed`` (layer files +
``mp_rank_*`` client state + optimizer shards, tag ``save_tag`` or ``global_step<N>``; ``latest``
is reserved) or ``huggingface`` (layer files then the DS→HF converter on rank 0).  LoRA
adapters are saved first and short-circuit the full save under ``only_save_trainable``.
"""
from __future__ import annotations

import os
import random

import numpy as np
import torch
import torch.distributed as dist

from ..parallel.grid import get_grid
from ..parallel.rng import get_rng_tracker
from ..utils.log import default_logger as logger


def _barrier():
    if dist.is_initialized():
        dist.barrier()


def get_checkpoint_name(path, iteration):
    g = get_grid()
    d = f"iter_{iteration:07d}"
    if g.pp == 1:
        return os.path.join(path, d, f"mp_rank_{g.tp_rank:02d}", "model_optim_rng.pt")
    return os.path.join(path, d, f"mp_rank_{g.tp_rank:02d}_{g.pp_rank:03d}", "model_optim_rng.pt")


def load_checkpoint(engine, optimizer, num_microbatches_calculator, cfg_loader, lora_mode=False, cfg_lora=None):
    """Returns (iteration, consumed_train_samples, consumed_train_tokens)."""
    it = samples = tokens = 0
    cfg_loader = cfg_loader or {}
    mode = cfg_loader.get("load_mode", "deepspeed")
    model = engine.module
    logger.info(f"Load Checkpoint in the {mode} Mode...")

    def maybe_lora():
        if lora_mode and cfg_lora and cfg_lora.get("loader"):
            from ..models.lora import load_lora_ckpt_pretrained
            load_lora_ckpt_pretrained(cfg_lora, model, optimizer)
            _barrier()

    if not cfg_loader.get("load_path") and not cfg_loader.get("debug"):
        logger.info("no loader.load_path: starting from the random initialisation")
        maybe_lora()
        return it, samples, tokens
    if mode != "deepspeed":
        from .hf_import import load_llama_from_hf_format
        load_llama_from_hf_format(model, cfg_loader.get("load_path"), cfg_loader.get("pretrain_type", "llama"),
                                  int(os.environ.get("LOADWORKER", cfg_loader.get("worker", 8))),
                                  cfg_loader.get("debug", False))
        if optimizer is not None and hasattr(optimizer, "refresh_fp32_params"):
            optimizer.refresh_fp32_params()
        _barrier()
        maybe_lora()
        return it, samples, tokens
    loaded, state = engine.load_checkpoint(cfg_loader["load_path"], tag=cfg_loader.get("load_tag"),
                                           load_optimizer_states=cfg_loader.get("load_optim", False),
                                           load_zero=cfg_loader.get("load_zero", False),
                                           load_lr_scheduler_states=False)
    if loaded is None:
        logger.info(f"WARNING: could not find the metadata file {cfg_loader['load_path']}; starting from random")
        return it, samples, tokens
    if cfg_loader.get("load_base_state", False):
        it = state.get("iteration", state.get("total_iters"))
        if it is None:
            raise KeyError("checkpoint metadata has no iteration")
        tokens = state.get("tokens", 0)
        samples = state.get("samples", 0)
        if num_microbatches_calculator is not None:
            num_microbatches_calculator.update(samples, True)
    if cfg_loader.get("load_rng_state", False):
        try:
            random.setstate(state["random_rng_state"])
            np.random.set_state(state["np_rng_state"])
            torch.set_rng_state(state["torch_rng_state"])
            if torch.cuda.is_available() and state.get("cuda_rng_state") is not None:
                torch.cuda.set_rng_state(state["cuda_rng_state"])
            if not state["rng_tracker_states"]:
                raise KeyError("rng_tracker_states")
            get_rng_tracker().set_states(state["rng_tracker_states"])
        except KeyError as e:
            raise KeyError(f"Unable to load rng state from checkpoint {cfg_loader['load_path']} ({e}); "
                           "set loader.load_rng_state: False to skip it") from e
    logger.info(f"Successfully loaded checkpoint from {cfg_loader['load_path']} at iteration {it}")
    _barrier()
    maybe_lora()
    return it, samples, tokens


def save_checkpoint(iteration, consumed_train_samples, consumed_train_tokens, engine, cfg_saver, lora_mode=False,
                    cfg_lora=None):
    _barrier()
    logger.info(f"saving checkpoint at iteration {iteration:7d} to {cfg_saver['save_path']}")
    model = engine.module
    if lora_mode and cfg_lora and cfg_lora.get("saver"):
        from ..models.lora import save_lora_ckpt_pretrained
        save_lora_ckpt_pretrained(cfg_lora, model, iteration=iteration)
        _barrier()
        if cfg_lora["saver"].get("only_save_trainable", False):
            return
    mode = cfg_saver.get("save_mode", "deepspeed")
    state = {"iteration": iteration, "samples": consumed_train_samples, "tokens": consumed_train_tokens}
    if cfg_saver.get("save_rng_state", False):
        state.update(random_rng_state=random.getstate(), np_rng_state=np.random.get_state(),
                     torch_rng_state=torch.get_rng_state(),
                     cuda_rng_state=torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
                     rng_tracker_states=get_rng_tracker().get_states())
    tag = cfg_saver.get("save_tag")
    if tag == "latest":
        raise ValueError("'latest' is reserved for the tag file; pick another save_tag")
    engine.save_checkpoint(cfg_saver["save_path"], tag=tag, client_state=state,
                           save_base_state=cfg_saver.get("save_base_state", True),
                           save_zero=cfg_saver.get("save_zero", False), save_optim=cfg_saver.get("save_optim", False))
    if mode == "huggingface" and get_grid().rank == 0:
        from .ds_to_hf import convert
        tag = tag or f"global_step{engine.global_steps}"
        a = model.args
        convert(os.path.join(cfg_saver["save_path"], tag), os.path.join(cfg_saver["save_path"], tag, "hf"),
                n_heads=a.num_attention_heads, num_key_value_heads=a.num_kv_attention_heads, norm_eps=a.norm_eps,
                rope_theta=a.rope_base, max_position_embeddings=a.seq_length or 2048)
    logger.info(f"Successfully saved checkpoint at iteration {iteration:7d} to {cfg_saver['save_path']}")
    _barrier()
