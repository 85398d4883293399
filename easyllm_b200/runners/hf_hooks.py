"""Hooks of the HF-style runner (llm/utils/general/hf_hook_helper.py:11-266).

``dynamic_checkpoint``: per iteration, choose how many decoder layers are recomputed from
the input size (``utils.dc_manager``).  ``hf_train_val_logger``: loss / accuracy entries of
the model output averaged over ranks, progress, epoch, lr, batch size, ETA; TensorBoard.
"""
from __future__ import annotations

import datetime
import time

import torch
import torch.distributed as dist

from ..config.registry import HOOK_REGISTRY
from ..utils.dc_manager import DynamicCheckpointManager
from ..utils.log import default_logger as logger
from .hooks import Hook, _tb_writer


@HOOK_REGISTRY.register("dynamic_checkpoint")
class DynamicCheckpointHook(Hook):
    def __init__(self, runner, enable=True, debug_freq=-1, strategy="memory_time", size_map=None,
                 level_keys=("layers",), **_):
        super().__init__(runner)
        self.enable = enable and size_map is not None
        self.mgr = None
        self.size_map, self.level_keys, self.debug_freq = size_map, level_keys, debug_freq

    def before_train(self):
        if self.enable:
            r = self.runner_ref()
            model = r.model.module if hasattr(r.model, "module") else r.model
            if hasattr(model, "gradient_checkpointing_disable"):
                model.gradient_checkpointing_disable()
            self.mgr = DynamicCheckpointManager(model, self.size_map, tuple(self.level_keys), debug=self.debug_freq > 0)

    def before_train_iter(self, cur_iter, batch=None):
        if self.mgr is not None and batch is not None:
            self.mgr.before_forward(batch["input_ids"])


@HOOK_REGISTRY.register("hf_train_val_logger")
class HFTrainValLoggerHook(Hook):
    def __init__(self, runner, freq=1, skip_first_k=1, tensorboard=False, log_dir="./log", logdir=None, summary_writer=None):
        super().__init__(runner)
        self.freq, self.skip = freq, skip_first_k
        self.writer = _tb_writer(logdir or log_dir) if tensorboard and (not dist.is_initialized() or dist.get_rank() == 0) else None
        self.t0 = None
        self.last_line = ""

    def before_train(self):
        self.t0, self.n = time.time(), 0

    def after_train_iter(self, cur_iter, output=None):
        r = self.runner_ref()
        if cur_iter - r.start_iter == self.skip:
            self.t0, self.n = time.time(), 0
        self.n += 1
        if (cur_iter + 1) % self.freq:
            return
        vals = {}
        for k, v in (output or {}).items():
            if "loss" in k or "accuracy" in k:
                t = v.detach().float().reshape(1).clone() if torch.is_tensor(v) else torch.tensor([float(v)])
                if dist.is_initialized() and dist.get_world_size() > 1:
                    t = t.to(r.device)
                    dist.all_reduce(t)
                    t /= dist.get_world_size()
                vals[k] = float(t)
        per = (time.time() - self.t0) / max(1, self.n)
        eta = datetime.timedelta(seconds=int(per * (r.train_iters - cur_iter - 1)))
        lr = r.optimizer.param_groups[0]["lr"]
        s = (f"Progress:[{100.0 * (cur_iter + 1) / r.train_iters:.1f}%][{cur_iter + 1}/{r.train_iters}] "
             f"Epoch:[{r.get_cur_train_epoch()}/{r.get_max_train_epoch()}] LR:{lr:.3E} "
             f"Batch:{r.global_train_batch_size} Time:{per:.3f}s ETA:{eta} "
             + " ".join(f"{k}:{v:.5f}" for k, v in vals.items()))
        logger.info(s)
        self.last_line = s
        if self.writer is not None:
            self.writer.add_scalar("train/lr", lr, cur_iter)
            for k, v in vals.items():
                self.writer.add_scalar(f"train/{k}", v, cur_iter)
