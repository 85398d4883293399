"""Training / evaluation engine: 1F1B pipeline schedule, gradient accumulation, ZeRO step.

This is the native counterpart of the DeepSpeed ``PipelineEngine`` contract the reference's
runner relies on (llm/runners/base_llm_runner.py:194-245, 367-410; hook_helper.py:122,177;
ckpt_helper.py:63-66,184-187): ``train_batch``, ``eval_batch``, ``set_batch_fn``,
``set_train_batch_size``, ``get_global_grad_norm``, ``optimizer.cur_scale``,
``fp16_enabled`` / ``bfloat16_enabled``, ``grid.get_*_parallel_rank``, ``save_checkpoint``
/ ``load_checkpoint`` (layer-file layout, see ``ckpt``).

Schedule (per ``train_batch``): stage ``s`` of ``P`` runs ``min(P − s − 1, M)`` warm-up
forwards, then alternates one forward / one backward, then drains the remaining backwards;
sends and receives of a steady-state slot are grouped so neighbouring stages never wait on
each other in opposite order.  Loss is the mean over micro-batches of each micro-batch's
own masked mean, averaged over DP and broadcast from the last stage.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..parallel.grid import get_grid
from .p2p import StageLink


class _GridView:
    """``engine.grid`` accessor names used by the runner."""

    def __init__(self, g):
        self._g = g

    def get_pipe_parallel_rank(self): return self._g.pp_rank
    def get_slice_parallel_rank(self): return self._g.tp_rank
    def get_data_parallel_rank(self): return self._g.dp_rank
    def get_pipe_parallel_world_size(self): return self._g.pp
    def get_slice_parallel_world_size(self): return self._g.tp
    def get_data_parallel_world_size(self): return self._g.dp


class PipelineEngine:
    def __init__(self, model, optimizer=None, lr_scheduler=None, config=None, batch_fn: Optional[Callable] = None):
        cfg = config or {}
        self.g = get_grid()
        self.grid = _GridView(self.g)
        self.module = model
        self.optimizer = optimizer
        self.lr_scheduler = lr_scheduler
        self.config = cfg
        self.batch_fn = batch_fn
        self.micro_batch_size = cfg.get("train_micro_batch_size_per_gpu", 1)
        self.micro_batches = cfg.get("gradient_accumulation_steps", 1)
        self.train_batch_size_ = cfg.get("train_batch_size", self.micro_batch_size * self.micro_batches * self.g.dp)
        self._fp16 = bool((cfg.get("fp16") or {}).get("enabled", False))
        self._bf16 = bool((cfg.get("bf16") or {}).get("enabled", False))
        self.global_steps = 0
        self.global_samples = 0
        self.skipped_steps = 0
        self.dtype = next(model.parameters()).dtype
        self.link = StageLink(self.dtype, dynamic=True) if self.g.pp > 1 else None
        self.total_loss = None
        self.fwd_outputs = []
        self._compute_loss = True        # set False by generation code that wants logits from eval_batch
        self.nvtx = bool(cfg.get("nvtx", False)) and torch.cuda.is_available()

    # ---- contract surface -------------------------------------------------------------------
    def fp16_enabled(self): return self._fp16
    def bfloat16_enabled(self): return self._bf16
    def set_batch_fn(self, fn): self.batch_fn = fn
    def is_first_stage(self): return self.g.is_first_stage()
    def is_last_stage(self): return self.g.is_last_stage()
    def train(self, mode=True): self.module.train(mode); return self
    def eval(self): self.module.eval(); return self

    def set_train_batch_size(self, n):
        per = self.micro_batch_size * self.g.dp
        if n % per:
            raise ValueError(f"train batch size {n} is not divisible by micro-batch × dp = {per}")
        self.train_batch_size_ = n
        self.micro_batches = n // per

    def get_global_grad_norm(self):
        return self.optimizer.get_global_grad_norm() if self.optimizer is not None else None

    def get_lr(self):
        return [pg["lr"] for pg in self.optimizer.param_groups]

    # ---- data -------------------------------------------------------------------------------
    def _next_batch(self, data_iter):
        """Only the first and last stage read data; returns (StageIO|None, labels|None)."""
        if not (self.g.is_first_stage() or self.g.is_last_stage()):
            return None, None
        batch = next(data_iter)
        if self.batch_fn is not None:
            batch = self.batch_fn(batch)
        inputs, labels = batch
        dev = next(self.module.parameters()).device

        def mv(t):
            return t.to(dev, non_blocking=True) if torch.is_tensor(t) else t
        io = None
        if self.g.is_first_stage():
            # parsed where the loader left the tensors (the host), then copied: no read-back from the GPU
            from ..models.llama import StageIO
            io = inputs if isinstance(inputs, StageIO) else self.module.parse_batch(inputs, device=dev)
        if self.g.is_last_stage() and labels is not None:
            labels = tuple(mv(t) for t in labels) if isinstance(labels, (tuple, list)) else (mv(labels),)
        else:
            labels = None
        return io, labels

    def _range(self, name):
        if self.nvtx:
            torch.cuda.nvtx.range_push(name)

    def _range_end(self):
        if self.nvtx:
            torch.cuda.nvtx.range_pop()

    # ---- single micro-batch pieces -------------------------------------------------------------
    def _forward(self, io, labels, train=True):
        self._range("forward")
        if io.hidden is not None and train:
            io.hidden.requires_grad_(True)
        inp = io.hidden
        out = self.module.forward_stage(io, labels)
        self._range_end()
        return inp, out

    def _backward(self, inp, out, grad):
        self._range("backward")
        if self.g.is_last_stage():
            scale = self.optimizer.cur_scale if self.optimizer is not None else 1.0
            (out * (scale / self.micro_batches)).backward()
        else:
            torch.autograd.backward(out.hidden, grad)
        self.optimizer.accumulate_grads()
        self._range_end()
        return inp.grad if inp is not None else None

    def _check_kernel_errors(self):
        """A fused kernel whose bounded wait on a peer expired returns with a partial result and an error code;
        refuse to apply an optimizer step computed from it (``ops.cuda.KernelError``)."""
        if next(self.module.parameters()).is_cuda:
            from ..ops import cuda as cu
            cu.check_step_errors()

    # ---- train --------------------------------------------------------------------------------
    def train_batch(self, data_iter=None, dynamic=True, sequence_parallel=None):
        if self.optimizer is None:
            raise RuntimeError("train_batch needs an optimizer")
        self.module.train()
        g, M, P = self.g, self.micro_batches, self.g.pp
        if self.link is not None:
            self.link.dynamic = dynamic
        losses = []
        if P == 1:
            for _ in range(M):
                io, labels = self._next_batch(data_iter)
                _, loss = self._forward(io, labels)
                self._backward(None, loss, None)
                losses.append(loss.detach())
        else:
            losses = self._train_1f1b(data_iter, M, P)
        self._check_kernel_errors()
        self._range("optimizer")
        stepped = self.optimizer.step()
        self._range_end()
        if not stepped:
            self.skipped_steps += 1
        self.global_steps += 1
        self.global_samples += self.train_batch_size_
        if self.lr_scheduler is not None and stepped:
            self.lr_scheduler.step(self.train_batch_size_)
        self.total_loss = self._aggregate_loss(losses)
        return self.total_loss

    def _train_1f1b(self, data_iter, M, P):
        """1F1B with asynchronous stage links: every send returns at once, and the receive of the next message of a
        direction is posted right after the send of the current one, so it lands while this stage computes."""
        g, link = self.g, self.link
        first, last = g.is_first_stage(), g.is_last_stage()
        warm = min(P - g.pp_rank - 1, M)
        steady = M - warm
        queue = []          # (input hidden, output) of forwards awaiting backward, FIFO
        losses = []
        n_fwd = n_bwd = 0

        def forward_one():
            nonlocal n_fwd
            io_in = link.wait_recv_fwd() if not first else None
            io, labels = self._next_batch(data_iter)
            if not first:
                io = io_in
            inp, out = self._forward(io, labels)
            queue.append((inp, out))
            n_fwd += 1
            if last:
                losses.append(out.detach())
            else:
                link.send_fwd(out)
            if not first and n_fwd < M:
                link.post_recv_fwd()                     # the next input travels during the compute that follows

        def backward_one():
            nonlocal n_bwd
            inp, o = queue.pop(0)
            grad = link.wait_recv_bwd(o.hidden) if not last else None
            dgrad = self._backward(inp, o, grad)
            n_bwd += 1
            if not first:
                link.send_bwd(dgrad)
            if not last and queue:
                link.post_recv_bwd(queue[0][1].hidden)   # gradient of the oldest forward still waiting

        if not first:
            link.post_recv_fwd()
        for _ in range(warm):
            forward_one()
        for _ in range(steady):
            forward_one()
            backward_one()
        for _ in range(warm):
            backward_one()
        link.flush()
        return losses

    def _aggregate_loss(self, losses):
        g = self.g
        dev = next(self.module.parameters()).device
        if g.is_last_stage() and losses:
            loss = torch.stack([l.float() for l in losses]).mean()
        else:
            loss = torch.zeros((), dtype=torch.float32, device=dev)
        if dist.is_initialized() and g.world > 1:
            if g.dp > 1 and g.is_last_stage():
                dist.all_reduce(loss, group=g.dp_group)
                loss = loss / g.dp
            if g.pp > 1:
                dist.broadcast(loss, g.last_stage_rank(), group=g.pp_group)
        return loss

    # ---- eval / inference ------------------------------------------------------------------------
    @torch.no_grad()
    def eval_batch(self, data_iter, compute_loss=True, reduce_output="avg", dynamic=True, sequence_parallel=None,
                   num_micro_batches=None, return_logits=False):
        """Forward-only pipeline pass.  With ``compute_loss`` returns the mean loss on every
        stage; otherwise the last stage returns its logits ``[b, s, V(/tp)]`` (others None)."""
        self.module.eval()
        compute_loss = compute_loss and self._compute_loss
        g, P = self.g, self.g.pp
        M = num_micro_batches or (self.micro_batches if compute_loss else 1)
        if self.link is not None:
            self.link.dynamic = dynamic
        outs = []
        for _ in range(M):
            io, labels = self._next_batch(data_iter)
            if P > 1 and not g.is_first_stage():
                io = self.link.wait_recv_fwd()
            out = self.module.forward_stage(io, labels if compute_loss else None,
                                            return_logits=not compute_loss)
            if P > 1 and not g.is_last_stage():
                self.link.send_fwd(out)
            elif g.is_last_stage():
                outs.append(out)
        if P > 1:
            self.link.flush()
        self.fwd_outputs = outs
        if compute_loss:
            return self._aggregate_loss(outs)
        if not g.is_last_stage():
            return None
        return outs[0] if M == 1 else outs

    @torch.no_grad()
    def forward_tokens(self, tokens, position_ids):
        """Inference forward of raw tokens through every stage (KV caches of the model are used
        when allocated).  Logits ``[b, s, V(/tp)]`` on the last stage, None elsewhere."""
        g = self.g
        io = None
        if g.is_first_stage():
            io = self.module.parse_batch((tokens, position_ids, None))
        if g.pp > 1 and not g.is_first_stage():
            self.link.dynamic = True
            io = self.link.wait_recv_fwd()
        out = self.module.forward_stage(io, None, return_logits=True)
        if g.pp > 1 and not g.is_last_stage():
            self.link.dynamic = True
            self.link.send_fwd(out)
            self.link.flush()
            return None
        return out

    # ---- checkpoint (delegated) ----------------------------------------------------------------------
    def save_checkpoint(self, save_dir, tag=None, client_state=None, save_base_state=True, save_zero=True,
                        save_optim=True):
        from ..ckpt.layer_files import save_engine_checkpoint
        return save_engine_checkpoint(self, save_dir, tag, client_state or {}, save_base_state, save_zero, save_optim)

    def load_checkpoint(self, load_dir, tag=None, load_optimizer_states=True, load_zero=True,
                        load_lr_scheduler_states=True, load_module_only=False):
        from ..ckpt.layer_files import load_engine_checkpoint
        return load_engine_checkpoint(self, load_dir, tag, load_optimizer_states and not load_module_only, load_zero,
                                      load_lr_scheduler_states and not load_module_only)


def initialize(model, optimizer=None, lr_scheduler=None, config=None, batch_fn=None):
    """``deepspeed.initialize`` counterpart: returns (engine, optimizer, None, lr_scheduler)."""
    zero_stage = ((config or {}).get("zero_optimization") or {}).get("stage", 0)
    if get_grid().pp > 1 and zero_stage >= 2:
        raise ValueError("ZeRO-2 is incompatible with pipeline parallelism (gradients of a stage are "
                         "accumulated over in-flight micro-batches); use stage 0/1 or pp=1")
    eng = PipelineEngine(model, optimizer, lr_scheduler, config, batch_fn)
    return eng, optimizer, None, lr_scheduler
