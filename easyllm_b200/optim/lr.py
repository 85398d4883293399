"""Learning-rate schedules (registry ``LR_REGISTRY``).

Parity: llm/utils/model/lr_helper.py:10-314.

* ``iter_base_annealing`` — progress is counted in **samples**: ``decay_steps = lr_decay_iters
  · global_batch_size`` and the engine steps the schedule by the global batch size each
  iteration; linear warm-up, then constant / linear / cosine decay to ``min_lr``.
* ``sample_base_annealing`` — warm-up counted in samples, decay counted in consumed tokens.
* ``hf_cosine`` — HuggingFace-style per-optimizer-step cosine with warm-up.

``state_dict`` keeps Megatron's keys (and accepts its legacy spellings) so schedules resume
from reference checkpoints.
"""
from __future__ import annotations

import math

from ..config.registry import LR_REGISTRY
from ..utils.log import default_logger as logger


def _decay_coeff(style, ratio):
    ratio = min(max(ratio, 0.0), 1.0)
    if style == "linear":
        return 1.0 - ratio
    if style == "cosine":
        return 0.5 * (math.cos(math.pi * ratio) + 1.0)
    raise ValueError(f"{style} decay style is not supported.")


class AnnealingLR:
    def __init__(self, optimizer, max_lr, min_lr, warmup_steps, decay_steps, decay_style, decay_tokens=None,
                 use_checkpoint_lr_scheduler=True, override_lr_scheduler=False):
        self.optimizer = optimizer
        self.max_lr, self.min_lr = float(max_lr), float(min_lr)
        if not 0.0 <= self.min_lr <= self.max_lr:
            raise ValueError("need 0 <= min_lr <= max_lr")
        if decay_steps <= 0 or warmup_steps >= decay_steps:
            raise ValueError("need 0 <= warmup_steps < decay_steps")
        self.warmup_steps, self.decay_steps, self.decay_style = warmup_steps, decay_steps, decay_style
        self.decay_tokens, self.num_steps, self.num_tokens, self.warmup_tokens = decay_tokens, 0, 0, 0
        if override_lr_scheduler and use_checkpoint_lr_scheduler:
            raise ValueError("both override and use-checkpoint are set.")
        self.override, self.use_ckpt = override_lr_scheduler, use_checkpoint_lr_scheduler

    def _apply(self):
        lr = self.get_lr()
        for group in self.optimizer.param_groups:
            group["lr"] = lr
        return lr

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"max_lr": self.max_lr, "warmup_steps": self.warmup_steps, "num_steps": self.num_steps,
                "warmup_tokens": self.warmup_tokens, "num_tokens": self.num_tokens,
                "decay_style": self.decay_style, "decay_steps": self.decay_steps, "min_lr": self.min_lr}

    def _pick(self, mine, saved, what):
        if self.override:
            logger.info(f" > overriding {what} value to {mine}")
            return mine
        if not self.use_ckpt and mine != saved:
            raise ValueError(f"AnnealingLR: class input value {mine} and checkpoint value {saved} for {what} do not match")
        return saved

    def load_state_dict(self, sd):
        get = lambda *names: next(sd[n] for n in names if n in sd)  # noqa: E731
        self.max_lr = self._pick(self.max_lr, get("start_lr", "max_lr"), "learning rate")
        self.min_lr = self._pick(self.min_lr, sd["min_lr"], "minimum learning rate")
        self.warmup_steps = self._pick(self.warmup_steps, get("warmup_iter", "warmup_steps"), "warmup iterations")
        self.decay_steps = self._pick(self.decay_steps, get("end_iter", "decay_steps"), "total number of iterations")
        self.decay_style = self._pick(self.decay_style, sd["decay_style"], "decay style")
        self.warmup_tokens = sd.get("warmup_tokens", self.warmup_tokens)
        self.num_tokens = sd.get("num_tokens", self.num_tokens)
        self.num_steps = 0
        self.step(get("num_iters", "num_steps"))


@LR_REGISTRY.register("iter_base_annealing")
class IterBaseAnnealingLR(AnnealingLR):
    def __init__(self, optimizer, max_lr, min_lr, decay_style, warmup_steps=None, decay_steps=None,
                 lr_decay_iters=None, train_iters=None, global_batch_size=None, lr_warmup_fraction=None,
                 lr_warmup_iters=None, decay_tokens=None, use_checkpoint_lr_scheduler=True,
                 override_lr_scheduler=False):
        if decay_steps is None:
            if lr_decay_iters is None:
                if train_iters is None:
                    raise ValueError("lr_decay_iters or train_iters is required")
                lr_decay_iters = train_iters
            decay_steps = lr_decay_iters * global_batch_size
        if warmup_steps is None:
            warmup_steps = lr_warmup_fraction * decay_steps if lr_warmup_fraction is not None \
                else (lr_warmup_iters or 0) * global_batch_size
        super().__init__(optimizer, max_lr, min_lr, warmup_steps, decay_steps, decay_style, decay_tokens,
                         use_checkpoint_lr_scheduler, override_lr_scheduler)
        self.step(0)

    def get_lr(self):
        if self.warmup_steps > 0 and self.num_steps <= self.warmup_steps:
            return self.max_lr * float(self.num_steps) / float(self.warmup_steps)
        if self.decay_style == "constant":
            return self.max_lr
        if self.num_steps > self.decay_steps:
            return self.min_lr
        ratio = float(self.num_steps - self.warmup_steps) / float(self.decay_steps - self.warmup_steps)
        return self.min_lr + _decay_coeff(self.decay_style, ratio) * (self.max_lr - self.min_lr)

    def step(self, increment=1):
        self.num_steps += increment
        self._apply()


@LR_REGISTRY.register("sample_base_annealing")
class SampleBaseAnnealingLR(AnnealingLR):
    def __init__(self, optimizer, max_lr, min_lr, decay_style, init_consumed_tokens=0, warmup_steps=None,
                 decay_steps=None, lr_decay_samples=None, train_samples=None, lr_warmup_fraction=None,
                 lr_warmup_samples=None, decay_tokens=None, use_checkpoint_lr_scheduler=True,
                 override_lr_scheduler=False):
        if decay_steps is None:
            decay_steps = lr_decay_samples if lr_decay_samples is not None else train_samples
            if decay_steps is None:
                raise ValueError("lr_decay_samples or train_samples is required")
        if warmup_steps is None:
            warmup_steps = lr_warmup_fraction * decay_steps if lr_warmup_fraction is not None else (lr_warmup_samples or 0)
        self.consumed_train_tokens = init_consumed_tokens
        super().__init__(optimizer, max_lr, min_lr, warmup_steps, decay_steps, decay_style, decay_tokens,
                         use_checkpoint_lr_scheduler, override_lr_scheduler)
        self.step(0)

    def get_lr(self):
        if self.warmup_steps > 0 and self.num_steps <= self.warmup_steps:
            if self.num_steps == self.warmup_steps and self.decay_tokens is not None:
                self.warmup_tokens = self.num_tokens
            return self.max_lr * float(self.num_steps) / float(self.warmup_steps)
        if self.decay_style == "constant":
            return self.max_lr
        if self.decay_tokens is None:
            raise ValueError("sample_base_annealing with a decaying style needs decay_tokens")
        if self.num_tokens > self.decay_tokens:
            return self.min_lr
        ratio = float(self.num_tokens - self.warmup_tokens) / float(self.decay_tokens - self.warmup_tokens)
        return self.min_lr + _decay_coeff(self.decay_style, ratio) * (self.max_lr - self.min_lr)

    def step(self, increment=1, token_num=None):
        self.num_tokens = self.consumed_train_tokens if token_num is None else token_num
        self.num_steps += increment
        self._apply()


@LR_REGISTRY.register("hf_cosine")
class HFCosineLR:
    """``lr = base · warmup_or_cosine(step)`` counted in optimizer steps."""

    def __init__(self, optimizer, warmup_steps, training_steps, last_epoch=-1, **_):
        self.optimizer, self.warmup_steps, self.training_steps = optimizer, warmup_steps, training_steps
        self.base_lrs = [g.get("initial_lr", g["lr"]) for g in optimizer.param_groups]
        for g, b in zip(optimizer.param_groups, self.base_lrs):
            g.setdefault("initial_lr", b)
        self.last_epoch = last_epoch
        self.step()

    def factor(self, step):
        if step < self.warmup_steps:
            return float(step) / float(max(1, self.warmup_steps))
        prog = float(step - self.warmup_steps) / float(max(1, self.training_steps - self.warmup_steps))
        return max(0.0, 0.5 * (1.0 + math.cos(math.pi * prog)))

    def step(self, increment=1):
        self.last_epoch += 1
        f = self.factor(self.last_epoch)
        for g, b in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = b * f

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"last_epoch": self.last_epoch, "base_lrs": self.base_lrs}

    def load_state_dict(self, sd):
        self.last_epoch = sd["last_epoch"] - 1
        self.base_lrs = sd.get("base_lrs", self.base_lrs)
        self.step()


def build_learning_rate_scheduler(cfg_lr, optimizer):
    cfg = {"type": cfg_lr["type"], "kwargs": dict(cfg_lr.get("kwargs") or {})}
    cfg["kwargs"]["optimizer"] = optimizer
    return LR_REGISTRY.build(cfg)
