"""Training hooks (registry ``HOOK_REGISTRY``; llm/utils/general/hook_helper.py:14-273).

Four hook points — ``before_train``, ``before_train_iter``, ``after_train_iter``,
``after_train`` — composed in config order; a ``train_val_logger`` is inserted when the
config has none.  Hooks keep a weak reference to the runner.

* ``train_val_logger``  per-iteration line: iteration, consumed samples / tokens, s/iter, lr,
  global batch, every ``*_loss`` averaged over the log window, loss scale (fp16), global grad
  norm, NaN/inf iteration count, samples/s, model TFLOPs (Megatron formula: coefficient 32 with
  a GLU MLP else 24; recompute factor 4 else 3), ETA; TensorBoard scalars when a writer is
  importable; periodic memory report.  Adds MFU against the measured bf16 peak when known.
* ``early_exit``  save-and-exit on wall-clock (agreed by an all-reduce MAX) or iteration limit.
* ``empty_cache`` / ``nan_guard`` (count | skip | abort policies are enforced by the optimizer;
  the hook aborts with a checkpoint after ``max_nan_iters`` bad iterations).
* ``watchdog``  host-side heartbeat monitor (see ``parallel.watchdog``).
"""
from __future__ import annotations

import datetime
import sys
import time
import weakref

import torch
import torch.distributed as dist

from ..config.registry import HOOK_REGISTRY
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger
from ..utils.timers import Timers, report_memory


class Hook:
    def __init__(self, runner):
        self.runner_ref = weakref.ref(runner)

    def before_train(self):
        pass

    def before_train_iter(self, cur_iter, batch=None):
        pass

    def after_train_iter(self, cur_iter, output=None):
        pass

    def after_train(self):
        pass

    def __call__(self, hook_type, *args, **kwargs):
        fn = getattr(self, hook_type)
        return fn(*args, **kwargs)


def _tb_writer(log_dir):
    for mod, cls in (("tensorboardX", "SummaryWriter"), ("torch.utils.tensorboard", "SummaryWriter")):
        try:
            m = __import__(mod, fromlist=[cls])
            return getattr(m, cls)(log_dir=log_dir)
        except Exception:
            continue
    return None


def model_flops_per_iteration(batch_size, seq_len, num_layers, hidden, vocab, glu=True, recompute=False):
    coeff = 32 if glu else 24
    factor = 4 if recompute else 3
    return (coeff * factor * batch_size * seq_len * num_layers * hidden ** 2) * (
        1.0 + seq_len / (6.0 * hidden) + vocab / (16.0 * num_layers * hidden))


@HOOK_REGISTRY.register("train_val_logger")
class TrainValLoggerHook(Hook):
    def __init__(self, runner, log_interval=1, report_memory_interval=10, log_params_norm=False, tensorboard=True,
                 log_dir="./log", peak_tflops=None):
        super().__init__(runner)
        self.timers = Timers()
        self.log_interval, self.report_memory_interval = log_interval, report_memory_interval
        self.losses, self.advanced, self.nan_iters = {}, 0, 0
        self.fp16 = runner.config["runtime"].get("fp16", False)
        self.writer = _tb_writer(log_dir) if tensorboard and get_grid().rank == 0 else None
        self.peak_tflops = peak_tflops
        self.last_line = ""

    def before_train(self):
        self.timers("train-iter-time").start()

    def after_train_iter(self, cur_iter, output=None):
        output = output or {}
        self.advanced += 1
        bad = False
        for k, v in output.items():
            if "_loss" in k:
                val = float(v.float().sum()) if torch.is_tensor(v) else float(v)
                self.losses[k] = self.losses.get(k, 0.0) + val
                bad = bad or val != val or val in (float("inf"), -float("inf"))
        self.nan_iters += int(bad)
        if (cur_iter + 1) % self.log_interval:
            return
        r = self.runner_ref()
        a = r.model.args
        g = get_grid()
        lr = r.optimizer.param_groups[0]["lr"]
        batch = r.micro_batch_size * g.dp * r.num_microbatches_calculator.get()
        per_iter = self.timers("train-iter-time").elapsed() / max(1, self.advanced)
        eta = datetime.timedelta(seconds=int(per_iter * (r.total_train_iters - cur_iter - 1)))
        flops = model_flops_per_iteration(batch, r.seq_length, a.num_layers, a.hidden_size, a.vocab_size,
                                          bool(a.glu_activation), a.checkpoint_activations and not a.dynamic_checkpoint)
        tflops = flops / (per_iter * g.world * 1e12)
        s = (f" iteration {cur_iter + 1:8d}/{r.total_train_iters:8d} | consumed samples: {r.consumed_train_samples:12d} |"
             f" consumed tokens: {r.consumed_train_tokens:12d} | elapsed time per iteration (s): {per_iter:.2f} |"
             f" learning rate: {lr:.3E} | global batch size: {batch:5d} |")
        if self.writer is not None:
            self.writer.add_scalar("train/lr", lr, cur_iter)
        for k in list(self.losses):
            avg = self.losses[k] / max(1, self.advanced)
            if avg > 0.0:
                s += f" {k}: {avg:.6E} |"
                if self.writer is not None:
                    self.writer.add_scalar(f"train/{k}", avg, cur_iter)
            self.losses[k] = 0.0
        if self.fp16:
            s += f" loss scale: {r.engine.optimizer.cur_scale:.1f} |"
        gn = r.engine.get_global_grad_norm()
        if gn is not None:
            s += f" grad norm: {gn:.3f} |"
        s += (f" number of nan iterations: {self.nan_iters:3d} | samples per second: {batch / per_iter:.3f} |"
              f" TFLOPs: {tflops:.2f} |")
        if self.peak_tflops:
            s += f" MFU: {100 * tflops / self.peak_tflops:.1f}% |"
        s += f" ETA Time: {eta}"
        logger.info(s)
        self.last_line = s
        self.advanced, self.nan_iters = 0, 0
        if cur_iter % self.report_memory_interval == 0 and lr > 0.0 and torch.cuda.is_available():
            report_memory(f"(after {cur_iter + 1} iterations)", logger.info)


@HOOK_REGISTRY.register("early_exit")
class EarlyExitHook(Hook):
    def __init__(self, runner, exit_duration_in_mins=None, exit_interval=None):
        super().__init__(runner)
        self.exit_duration_in_mins, self.exit_interval = exit_duration_in_mins, exit_interval

    def _save_and_exit(self, cur_iter, why):
        r = self.runner_ref()
        r.save_checkpoint(cur_iter + 1)
        logger.info(f"Exiting program {why}")
        sys.exit()

    def after_train_iter(self, cur_iter, output=None):
        r = self.runner_ref()
        if self.exit_duration_in_mins is not None:
            mins = (time.time() - r.start_time) / 60.0
            flag = torch.tensor([int(mins > self.exit_duration_in_mins)], dtype=torch.int32, device=r.device)
            if dist.is_initialized():
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            if int(flag):
                self._save_and_exit(cur_iter, f"after {mins:.1f} minutes")
        if self.exit_interval and (cur_iter + 1) % self.exit_interval == 0:
            self._save_and_exit(cur_iter, f"at iteration {cur_iter + 1}")


@HOOK_REGISTRY.register("empty_cache")
class EmptyCacheHook(Hook):
    def __init__(self, runner, freq=1):
        super().__init__(runner)
        self.freq = freq

    def after_train_iter(self, cur_iter, output=None):
        if cur_iter % self.freq == 0 and cur_iter > 0 and torch.cuda.is_available():
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats()


@HOOK_REGISTRY.register("nan_guard")
class NanGuardHook(Hook):
    """Abort with a checkpoint after ``max_nan_iters`` consecutive non-finite losses."""

    def __init__(self, runner, max_nan_iters=5, save=True):
        super().__init__(runner)
        self.max_nan_iters, self.save, self.streak = max_nan_iters, save, 0

    def after_train_iter(self, cur_iter, output=None):
        val = float((output or {}).get("lm_loss", 0.0))
        self.streak = self.streak + 1 if (val != val or abs(val) == float("inf")) else 0
        if self.streak >= self.max_nan_iters:
            r = self.runner_ref()
            if self.save:
                r.save_checkpoint(cur_iter + 1)
            raise FloatingPointError(f"{self.streak} consecutive non-finite losses at iteration {cur_iter + 1}")


class ComposeHook:
    def __init__(self, hooks):
        self._hooks = list(hooks)

    def __call__(self, hook_type, *args, **kwargs):
        for h in self._hooks:
            h(hook_type, *args, **kwargs)

    def __iter__(self):
        return iter(self._hooks)


def build_hooks(runner, cfg_hooks, add_log_if_not_exists=True):
    cfg_hooks = list(cfg_hooks or [])
    if add_log_if_not_exists and not any("train_val_logger" in c["type"] for c in cfg_hooks):
        cfg_hooks.insert(0, {"type": "train_val_logger", "kwargs": {}})
    hooks = []
    for c in cfg_hooks:
        kw = dict(c.get("kwargs") or {})
        kw["runner"] = runner
        hooks.append(HOOK_REGISTRY.build({"type": c["type"], "kwargs": kw}))
    return ComposeHook(hooks)


@HOOK_REGISTRY.register("watchdog")
class WatchdogHook(Hook):
    """Heartbeat monitor: raises ``RankFailure`` on the training thread (between steps) when a peer
    stops beating; optionally saves a checkpoint first."""

    def __init__(self, runner, interval=5.0, timeout=120.0, port=None, save_on_failure=False, check_device_flag=True):
        super().__init__(runner)
        self.kw = dict(interval=interval, timeout=timeout, port=port, check_device_flag=check_device_flag)
        self.save_on_failure = save_on_failure
        self.wd = None

    def before_train(self):
        from ..parallel.watchdog import Watchdog
        g = get_grid()
        if g.world > 1:
            self.wd = Watchdog(g.rank, g.world, **self.kw).start()

    def after_train_iter(self, cur_iter, output=None):
        if self.wd is not None:
            self.wd.check()

    def after_train(self):
        if self.wd is not None:
            self.wd.leave()


@HOOK_REGISTRY.register("torch_profiler")
class TorchProfilerHook(Hook):
    """Optional ``torch.profiler`` window over a few training iterations (the reference has no profiler
    integration; its only timers are the wall-clock ``Timers`` of the logger hook).

    Skips ``wait`` iterations, warms the profiler for ``warmup``, records ``active`` iterations, then writes a Chrome
    trace ``<out_dir>/trace_rank<r>_iter<i>.json`` and a text table of the top operators; ``ranks`` limits which
    global ranks profile (default rank 0 only).  CUDA activity is recorded when a GPU is present.
    """

    def __init__(self, runner, out_dir="profiler", wait=2, warmup=1, active=2, repeat=1, ranks=(0,),
                 record_shapes=False, with_stack=False, profile_memory=False, row_limit=30):
        super().__init__(runner)
        self.out_dir, self.ranks, self.row_limit = out_dir, tuple(ranks), row_limit
        self.sched = dict(wait=wait, warmup=warmup, active=active, repeat=repeat)
        self.opts = dict(record_shapes=record_shapes, with_stack=with_stack, profile_memory=profile_memory)
        self.prof = None
        self.written = []

    def _on_ready(self, prof):
        import os
        os.makedirs(self.out_dir, exist_ok=True)
        rank = get_grid().rank if torch.distributed.is_initialized() else 0
        base = os.path.join(self.out_dir, f"trace_rank{rank}_iter{self._iter}")
        prof.export_chrome_trace(base + ".json")
        key = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
        with open(base + ".txt", "w") as f:
            f.write(prof.key_averages().table(sort_by=key, row_limit=self.row_limit))
        self.written.append(base + ".json")
        logger.info(f"torch.profiler trace written to {base}.json")

    def before_train(self):
        from torch.profiler import ProfilerActivity, profile, schedule
        rank = get_grid().rank if torch.distributed.is_initialized() else 0
        if rank not in self.ranks:
            return
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
        self._iter = 0
        self.prof = profile(activities=acts, schedule=schedule(**self.sched), on_trace_ready=self._on_ready, **self.opts)
        self.prof.__enter__()

    def after_train_iter(self, cur_iter, output=None):
        if self.prof is not None:
            self._iter = cur_iter
            self.prof.step()

    def after_train(self):
        if self.prof is not None:
            self.prof.__exit__(None, None, None)
            self.prof = None
