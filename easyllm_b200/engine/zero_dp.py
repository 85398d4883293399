"""Single-axis data-parallel engine for module-tree (HF-style) models.

What the HF runner of the reference gets from ``deepspeed.initialize`` with ZeRO-1/2, or from
DDP + GradScaler without it (llm/runners/hf_runner.py:150-170, 238-278): ``backward(loss)``
accumulates, ``step()`` acts on accumulation boundaries.  Parameters live in the flat buffers
of ``ZeroOptimizer`` over the whole world as the DP group: gradients are reduce-scattered,
the fp32 Adam shard is updated by the fused kernel and parameters are all-gathered (on GPUs by
the two fused kernels of ``ops/csrc/zero_fused.cu``).  Stages 1 and 2 share this path: gradients
are accumulated in fp32 over the micro-batches and reduced once per optimizer step.
"""
from __future__ import annotations

import torch.distributed as dist

from ..optim.zero import ZeroOptimizer
from ..parallel.grid import get_grid


class ZeroDPEngine:
    def __init__(self, model, optimizer: ZeroOptimizer, lr_scheduler=None, config=None):
        cfg = config or {}
        self.module, self.optimizer, self.lr_scheduler, self.config = model, optimizer, lr_scheduler, cfg
        self.gradient_accumulation_steps = int(cfg.get("gradient_accumulation_steps", 1))
        self.micro_steps = 0
        self.global_steps = 0
        self.skipped_steps = 0
        self._fp16 = bool((cfg.get("fp16") or {}).get("enabled", False))
        self._bf16 = bool((cfg.get("bf16") or {}).get("enabled", False))

    def __call__(self, *a, **k):
        return self.module(*a, **k)

    def train(self, mode=True):
        self.module.train(mode)
        return self

    def eval(self):
        self.module.eval()
        return self

    def fp16_enabled(self): return self._fp16
    def bfloat16_enabled(self): return self._bf16
    def get_global_grad_norm(self): return self.optimizer.get_global_grad_norm()
    def is_gradient_accumulation_boundary(self): return (self.micro_steps + 1) % self.gradient_accumulation_steps == 0

    def backward(self, loss):
        scale = self.optimizer.cur_scale / self.gradient_accumulation_steps
        (loss * scale).backward()
        self.optimizer.accumulate_grads()

    def step(self):
        boundary = self.is_gradient_accumulation_boundary()
        self.micro_steps += 1
        if not boundary:
            return False
        if next(self.module.parameters()).is_cuda:
            from ..ops import cuda as cu
            cu.check_step_errors()           # a kernel that gave up a bounded wait left a partial result: do not apply it
        ok = self.optimizer.step()
        self.global_steps += 1
        if not ok:
            self.skipped_steps += 1
        elif self.lr_scheduler is not None:
            self.lr_scheduler.step()
        return ok

    # ---- checkpoints: <dir>/<tag>/mp_rank_00_model_states.pt + zero shards -------------------------
    def save_checkpoint(self, save_dir, tag=None, client_state=None):
        import os
        from ..ckpt.layer_files import atomic_save, zero_file
        g = get_grid()
        tag = tag or f"global_step{self.global_steps}"
        d = os.path.join(save_dir, tag)
        os.makedirs(d, exist_ok=True)
        if g.rank == 0:
            state = {"module": {k: v.detach().cpu() for k, v in self.module.state_dict().items()},
                     "global_steps": self.global_steps, "micro_steps": self.micro_steps,
                     "lr_scheduler": self.lr_scheduler.state_dict() if self.lr_scheduler is not None else None,
                     "dp_world_size": g.world}
            state.update(client_state or {})
            atomic_save(state, os.path.join(d, "mp_rank_00_model_states.pt"))
        atomic_save({"optimizer_state_dict": self.optimizer.state_dict()}, zero_file(d, g.rank, 0, self._bf16))
        if dist.is_initialized():
            dist.barrier()
        if g.rank == 0:
            with open(os.path.join(save_dir, "latest"), "w") as f:
                f.write(tag)

    def load_checkpoint(self, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True):
        import os
        from ..ckpt.layer_files import read_latest, safe_load, zero_file
        g = get_grid()
        tag = tag or read_latest(load_dir)
        if tag is None:
            return None, {}
        d = os.path.join(load_dir, tag)
        state = safe_load(os.path.join(d, "mp_rank_00_model_states.pt"))
        self.module.load_state_dict(state["module"])
        self.optimizer.refresh_fp32_params()
        self.global_steps, self.micro_steps = state.get("global_steps", 0), state.get("micro_steps", 0)
        if load_lr_scheduler_states and self.lr_scheduler is not None and state.get("lr_scheduler"):
            self.lr_scheduler.load_state_dict(state["lr_scheduler"])
        if load_optimizer_states:
            f = zero_file(d, g.rank, 0, self._bf16)
            if os.path.exists(f) and state.get("dp_world_size") == g.world:
                self.optimizer.load_state_dict(safe_load(f)["optimizer_state_dict"])
        return d, {k: v for k, v in state.items() if k != "module"}
