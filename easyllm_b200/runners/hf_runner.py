"""HuggingFace-style data-parallel runner: ``python -m easyllm_b200.runners.hf_runner --config x.yaml``.

Parity: llm/runners/hf_runner.py:34-332 and llm/utils/general/{hf_build_utils,hf_utils}.py —
tokenizer → model (registry, optional LoRA adapters, gradient checkpointing unless a Dynamic
Checkpoint hook manages it) → hooks → data (collator forced to ``offset_label=False``: these
models shift labels themselves; ``dist`` / ``dist_test`` samplers) → optimizer + LR schedule →
ZeRO-1/2 engine (``deepspeed.enabled``) or plain DP with a sharded grad scaler → checkpoints
(``deepspeed``: ``global_step<N>`` + world-size check; ``huggingface``: ``checkpoint-<step>/``
via ``save_pretrained`` + tokenizer).  ``infer()`` runs interactive / eval generation.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..config import load_yaml, parse_args
from ..config.registry import MODULE_ZOO_REGISTRY
from ..data import build_dataset, build_tokenizer
from ..data.loader import build_batch_collator, build_data_loader
from ..data.samplers import build_batch_sampler
from ..engine.zero_dp import ZeroDPEngine
from ..optim import build_learning_rate_scheduler, build_optimizer
from ..optim.grad_scaler import ShardedGradScaler
from ..parallel.grid import initialize_distributed
from ..utils.log import default_logger as logger
from . import hf_hooks  # noqa: F401
from .hooks import build_hooks


def hack_model(model):
    """Frozen embeddings + checkpointing: make embedding outputs require grad so recomputed blocks
    still receive gradients (hf_build_utils.py:30-46)."""
    emb = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else None
    if emb is not None:
        emb.register_forward_hook(lambda m, i, o: o.requires_grad_(True))


def build_hf_model(cfg_model):
    from ..models import hf_models  # noqa: F401  (fills the zoo)
    model = MODULE_ZOO_REGISTRY.build({"type": cfg_model["type"], "kwargs": dict(cfg_model.get("kwargs") or {})})
    peft = cfg_model.get("peft_model_cfg")
    if peft:
        from ..models.hf_models.lora import add_lora, load_adapter
        if peft.get("peft_path"):                      # continue from / serve a saved adapter
            load_adapter(model, peft["peft_path"])
            logger.info(f"load peft model from : {peft['peft_path']}")
        else:
            add_lora(model, peft)
    return model


class HFRunner:
    def __init__(self, args, cfg=None, training=True):
        self.args, self.config, self.training = args, cfg, training
        cfg.setdefault("runtime", {})
        ds = cfg.get("deepspeed") or {}
        self.deepspeed = ds.get("enabled", False)
        dcfg = ds.get("config") or {}
        self.ds_config = dcfg
        self.dtype = torch.bfloat16 if (dcfg.get("bf16") or {}).get("enabled") else \
            torch.float16 if (dcfg.get("fp16") or {}).get("enabled") else torch.float32
        self.gradient_accumulation_steps = cfg["runtime"].get("gradient_accumulation_steps", 1)
        self.start_iter = self.cur_iter = 0
        self.build()

    def build(self):
        self.build_env()
        self.tokenizer = build_tokenizer(self.config["tokenizer"])
        self.build_model()
        self._hooks = build_hooks(self, self.config.get("hooks", []) if self.training else [], False)
        self.build_data()
        self.build_trainer()
        self.load_checkpoints(self.config.get("loader") or {})

    def build_env(self):
        import random
        import numpy as np
        if not dist.is_initialized() and int(os.environ.get("WORLD_SIZE", "1")) > 1:
            initialize_distributed(1, 1, backend=getattr(self.args, "distributed_backend", "nccl"),
                                   launcher=getattr(self.args, "launcher", "torch"))
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        seed = self.config["runtime"].get("seed", 42) + 100 * self.rank
        random.seed(seed); np.random.seed(seed); torch.manual_seed(seed)
        self.device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")

    def build_model(self):
        model = build_hf_model(self.config["model"])
        use_dc = any(h["type"] == "dynamic_checkpoint" for h in self.config.get("hooks", []))
        if self.config["runtime"].get("gradient_checkpointing", True) and not use_dc and self.training:
            model.gradient_checkpointing_enable()
            if self.config["model"].get("peft_model_cfg") is not None:
                hack_model(model)
        self.model = model.to(self.device)
        if self.dtype != torch.float32 and self.training:
            self.model = self.model.to(self.dtype)

    def build_data(self):
        self.data_loaders = {}
        for dt in self.config["data"].get("data_types", []):
            c = self.config["data"][dt]
            ds = build_dataset(c["dataset"], self.tokenizer)
            cc = {"type": c["batch_collector"]["type"], "kwargs": dict(c["batch_collector"].get("kwargs") or {})}
            if cc["type"] == "batch_align":
                cc["kwargs"]["offset_label"] = False
            coll = build_batch_collator(cc, self.tokenizer)
            bs = c["batch_sampler"]
            bk = dict(bs.get("kwargs") or {})
            sampler = dict(bk.get("sampler") or {"type": "dist"})
            if dt in ("val", "test"):
                sampler["type"] = "dist_test"
            bcfg = {"type": bs.get("type", "base"),
                    "kwargs": {"sampler": sampler, "total_samples": len(ds), "data_parallel_rank": self.rank,
                               "data_parallel_size": self.world,
                               "micro_batch_size": bk.get("batch_size", bk.get("micro_batch_size", 1))}}
            self.data_loaders[dt] = build_data_loader(c.get("data_loader", {"type": "base"}), ds,
                                                      build_batch_sampler(bcfg), coll)

    def build_trainer(self):
        self.global_train_batch_size = 1
        if not self.training:
            return
        tr = self.config["trainer"]
        self.train_iters = tr["train_iters"]
        self.save_interval = (self.config.get("saver") or {}).get("save_interval", 100)
        loader = self.data_loaders["train"]
        self.mirco_train_batch_size = loader.batch_sampler.batch_size
        self.train_epoch_size = max(1, loader.get_epoch_size() // self.gradient_accumulation_steps)
        self.global_train_batch_size = self.mirco_train_batch_size * self.world * self.gradient_accumulation_steps
        stage = (self.ds_config.get("zero_optimization") or {}).get("stage", 1) if self.deepspeed else 0
        # `trainer.optimizer.type`: Adam / AdamW / FusedAdam run on the native ZeRO optimizer, every other type
        # (SophiaG, Adam8bit, SGD, torch.optim.*) on the wrapped torch optimizer with plain data parallelism
        cfg_optim = {"type": tr["optimizer"].get("type", "AdamW"), "kwargs": dict(tr["optimizer"].get("kwargs") or {})}
        self.optimizer = build_optimizer(cfg_optim, self.model, zero_stage=stage,
                                         grad_clip=self.ds_config.get("gradient_clipping", 0.0),
                                         fp16=self.dtype == torch.float16, engine_contract=True)
        lr_cfg = {"type": tr["lr_scheduler"]["type"], "kwargs": dict(tr["lr_scheduler"].get("kwargs") or {})}
        self.lr_scheduler = build_learning_rate_scheduler(lr_cfg, self.optimizer)
        self.engine = ZeroDPEngine(self.model, self.optimizer, self.lr_scheduler,
                                   dict(self.ds_config, gradient_accumulation_steps=self.gradient_accumulation_steps))
        # fp16 loss scaling lives in the optimizer (``optimizer.cur_scale``; an overflowing step is skipped and the
        # scale halved) with and without the ZeRO engine; ``ShardedGradScaler`` stays available to user loops
        self.scaler = None

    def get_cur_train_epoch(self):
        return self.cur_iter // self.train_epoch_size + 1

    def get_max_train_epoch(self):
        return max(self.train_iters - 1, 1) // self.train_epoch_size + 1

    # ---- checkpoints ---------------------------------------------------------------------------------
    def load_checkpoints(self, cfg):
        if not cfg.get("enabled", False) or not cfg.get("load_path"):
            return
        mode = cfg.get("load_mode", "huggingface")
        if mode == "deepspeed":
            _, client = self.engine.load_checkpoint(cfg["load_path"], cfg.get("load_tag"),
                                                    cfg.get("load_optim", True))
            if client.get("world_size") not in (None, self.world):
                raise ValueError("deepspeed-mode resume needs the world size the checkpoint was saved with")
            self.start_iter = client.get("iteration", self.engine.global_steps)
            bs = self.data_loaders["train"].batch_sampler
            if hasattr(bs, "set_consumed_samples"):
                bs.set_consumed_samples(self.start_iter * self.global_train_batch_size)
        elif mode == "huggingface":
            from ..ckpt.hf_import import load_hf_state
            from ..models.hf_models.io import import_state
            sd = import_state(load_hf_state(cfg["load_path"]), self.model.arch)
            own = set(self.model.state_dict())
            # a LoRA-wrapped projection keeps its frozen weight one level down (`q_proj.base.weight`)
            sd = {(k if k in own else k.replace(".weight", ".base.weight").replace(".bias", ".base.bias")): v.to(self.dtype)
                  for k, v in sd.items()}
            missing, unexpected = self.model.load_state_dict(sd, strict=False)
            tied = getattr(self.model.arch, "tie_word_embeddings", False)
            missing = [m for m in missing if "lora_" not in m and not (tied and m == "lm_head.weight")]
            if missing or unexpected:
                raise RuntimeError(f"{cfg['load_path']}: missing {missing[:8]}, unexpected {unexpected[:8]}")
            if self.training:
                self.optimizer.refresh_fp32_params()
        else:
            raise NotImplementedError(mode)

    def save_checkpoint(self, cfg, global_step):
        if not cfg.get("enabled", True):
            return
        path = cfg.get("save_path", "checkpoints")
        if cfg.get("save_mode", "deepspeed") == "huggingface":
            if self.rank == 0:
                out = os.path.join(path, f"checkpoint-{global_step}")
                if getattr(self.model, "peft_config", None):
                    # a LoRA run saves what peft's save_pretrained saves: the adapter tensors and their config
                    from ..models.hf_models.lora import save_adapter
                    save_adapter(self.model, out)
                else:
                    self.model.save_pretrained(out)
                if hasattr(self.tokenizer, "save_pretrained"):
                    self.tokenizer.save_pretrained(out)
        else:
            self.engine.save_checkpoint(path, f"global_step{global_step}",
                                        {"iteration": global_step, "world_size": self.world})
        if dist.is_initialized():
            dist.barrier()

    # ---- loops -------------------------------------------------------------------------------------------
    def get_batch(self, kind="train"):
        if not hasattr(self, "data_iterators"):
            self.data_iterators = {}
        it = self.data_iterators.get(kind)
        if it is None:
            it = self.data_iterators[kind] = iter(self.data_loaders[kind])
        try:
            batch = next(it)
        except StopIteration:
            it = self.data_iterators[kind] = iter(self.data_loaders[kind])
            batch = next(it)
        # the batch stays on the host: the model parses it there (document boundaries, longest document, highest
        # position) and copies what the kernels need, so no micro-batch waits for a read-back from the GPU
        batch = dict(batch)
        batch.setdefault("position_ids", None)
        batch.setdefault("cu_seqlens", None)
        return batch

    def train(self):
        self.model.train()
        self._hooks("before_train")
        gas = self.gradient_accumulation_steps
        output = {}
        for it in range(self.start_iter * gas, self.train_iters * gas):
            self.cur_iter = it // gas
            batch = self.get_batch()
            self._hooks("before_train_iter", self.cur_iter, batch)
            output = self.model(batch["input_ids"], batch["attention_mask"], labels=batch["labels"],
                                position_ids=batch["position_ids"], cu_seqlens=batch["cu_seqlens"])
            loss = sum(v for k, v in output.items() if "loss" in k)
            self.engine.backward(loss)
            self.engine.step()
            if (it + 1) % gas == 0:
                if (self.cur_iter + 1) % self.save_interval == 0:
                    self.save_checkpoint(self.config.get("saver", {}), self.cur_iter + 1)
                self._hooks("after_train_iter", self.cur_iter, output)
        saver = dict(self.config.get("saver", {}))
        if saver.get("save_path"):
            saver["save_mode"] = "huggingface"
            self.save_checkpoint(saver, self.train_iters)
        self._hooks("after_train")
        return output

    def infer(self):
        from ..infer.hf_inference import hf_inference
        self.model.eval()
        hf_inference(self.config.get("infer_cfg", {}), self.model, self.tokenizer, self.config.get("infer_tokenization"),
                     self.device, self.args)


def main(argv=None):
    args = parse_args(argv)
    cfg = load_yaml(args.config)
    runner = HFRunner(args, cfg, training=not args.inference)
    runner.infer() if args.inference else runner.train()


if __name__ == "__main__":
    main()
