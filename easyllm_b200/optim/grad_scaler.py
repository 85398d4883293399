"""Shard-aware dynamic loss scaler for fp16 training without the ZeRO engine.

Parity: llm/utils/general/grad_scaler.py:72-417 (fairscale / FSDP style): ``scale(loss)``,
``unscale_(optimizer)``, ``step(optimizer)``, ``update()``; works with CPU gradients; the
``found_inf`` flag is all-reduced (MAX) over the process group so every shard skips the same
step.  Written directly on tensors instead of subclassing ``torch.cuda.amp.GradScaler``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class ShardedGradScaler:
    def __init__(self, init_scale=2.0 ** 16, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000,
                 enabled=True, process_group=None):
        self._enabled = enabled
        self._scale = float(init_scale)
        self.growth_factor, self.backoff_factor, self.growth_interval = growth_factor, backoff_factor, growth_interval
        self._growth_tracker = 0
        self.group = process_group
        self._found_inf = {}
        self._unscaled = set()

    def is_enabled(self):
        return self._enabled

    def get_scale(self):
        return self._scale if self._enabled else 1.0

    def scale(self, outputs):
        if not self._enabled:
            return outputs
        if torch.is_tensor(outputs):
            return outputs * self._scale
        return type(outputs)(self.scale(o) for o in outputs)

    def _grads(self, optimizer):
        for g in optimizer.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    yield p.grad

    def unscale_(self, optimizer):
        if not self._enabled or id(optimizer) in self._unscaled:
            return
        inv = 1.0 / self._scale
        found = 0.0
        for grad in self._grads(optimizer):
            grad.mul_(inv)
            if not bool(torch.isfinite(grad).all()):
                found = 1.0
        flag = torch.tensor([found])
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else "cpu"
            flag = flag.to(dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        self._found_inf[id(optimizer)] = float(flag) > 0
        self._unscaled.add(id(optimizer))

    def step(self, optimizer, *a, **k):
        if not self._enabled:
            return optimizer.step(*a, **k)
        self.unscale_(optimizer)
        if self._found_inf.get(id(optimizer), False):
            return None
        return optimizer.step(*a, **k)

    def update(self, new_scale=None):
        if not self._enabled:
            return
        if new_scale is not None:
            self._scale = float(new_scale)
        elif any(self._found_inf.values()):
            self._scale *= self.backoff_factor
            self._growth_tracker = 0
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self.growth_interval:
                self._scale *= self.growth_factor
                self._growth_tracker = 0
        self._found_inf.clear()
        self._unscaled.clear()

    def state_dict(self):
        return {"scale": self._scale, "growth_factor": self.growth_factor, "backoff_factor": self.backoff_factor,
                "growth_interval": self.growth_interval, "_growth_tracker": self._growth_tracker} if self._enabled else {}

    def load_state_dict(self, sd):
        if sd:
            self._scale, self._growth_tracker = sd["scale"], sd["_growth_tracker"]
