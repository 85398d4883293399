"""Pipeline-stage point-to-point exchange of activations and gradients.

Stays on ``torch.distributed`` p2p (NCCL on GPUs, gloo on CPU) by design: a stage boundary
moves one ``[T/tp, h]`` tensor per micro-batch, which the 1F1B schedule overlaps with
compute.  ``dynamic=True`` re-negotiates the shape of every forward message with a small
header (micro-batches of different token counts: ``runtime.dynamic`` in the reference,
llm/runners/base_llm_runner.py:240-242); otherwise the first header is cached.

One forward message = header int64[8] (dynamic only) + hidden ``[T_local, h]`` + int32 meta
``[T + n_cu]`` (position ids, then cu_seqlens).  Backward messages are the hidden gradient.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..models.llama import StageIO
from ..parallel.grid import get_grid

_HDR = 8


def _dev():
    if dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


class StageLink:
    def __init__(self, dtype, dynamic=True):
        self.g = get_grid()
        self.dtype = dtype
        self.dynamic = dynamic
        self._cached_hdr = None

    # ---- helpers --------------------------------------------------------------------------
    def _header_of(self, io: StageIO):
        ncu = 0 if io.cu_seqlens is None else io.cu_seqlens.numel()
        return torch.tensor([io.hidden.shape[0], io.hidden.shape[1], io.batch, io.seq, io.max_seqlen,
                             io.max_position, ncu, io.position_ids.numel()], dtype=torch.int64)

    def _meta_of(self, io: StageIO):
        parts = [io.position_ids.to(torch.int32)]
        if io.cu_seqlens is not None:
            parts.append(io.cu_seqlens.to(torch.int32))
        return torch.cat(parts).contiguous()

    def _run(self, ops):
        if not ops:
            return
        for w in dist.batch_isend_irecv(ops):
            w.wait()

    # ---- the combined exchange ------------------------------------------------------------------
    def exchange(self, send_fwd: Optional[StageIO] = None, recv_fwd: bool = False,
                 send_bwd: Optional[torch.Tensor] = None, recv_bwd_like: Optional[torch.Tensor] = None):
        """Send/receive in one grouped call.  Returns (StageIO or None, grad tensor or None)."""
        g = self.g
        nxt, prv = g.next_stage_rank(), g.prev_stage_rank()
        dev = _dev()
        hdr_in = None
        # phase 1: headers for the forward direction
        need_hdr = self.dynamic or self._cached_hdr is None
        ops = []
        if send_fwd is not None and (self.dynamic or not getattr(self, "_sent_hdr", False)):
            ops.append(dist.P2POp(dist.isend, self._header_of(send_fwd).to(dev), nxt))
            self._sent_hdr = True
        if recv_fwd and need_hdr:
            hdr_in = torch.empty(_HDR, dtype=torch.int64, device=dev)
            ops.append(dist.P2POp(dist.irecv, hdr_in, prv))
        self._run(ops)
        if recv_fwd:
            if hdr_in is not None:
                self._cached_hdr = hdr_in.cpu().tolist()
            hdr = self._cached_hdr
        # phase 2: payloads
        ops = []
        hidden_in = meta_in = grad_in = None
        if send_fwd is not None:
            ops.append(dist.P2POp(dist.isend, send_fwd.hidden.detach().contiguous(), nxt))
            ops.append(dist.P2POp(dist.isend, self._meta_of(send_fwd).to(dev), nxt))
        if recv_fwd:
            hidden_in = torch.empty(hdr[0], hdr[1], dtype=self.dtype, device=dev)
            meta_in = torch.empty(hdr[7] + hdr[6], dtype=torch.int32, device=dev)
            ops.append(dist.P2POp(dist.irecv, hidden_in, prv))
            ops.append(dist.P2POp(dist.irecv, meta_in, prv))
        if send_bwd is not None:
            ops.append(dist.P2POp(dist.isend, send_bwd.contiguous(), prv))
        if recv_bwd_like is not None:
            grad_in = torch.empty_like(recv_bwd_like)
            ops.append(dist.P2POp(dist.irecv, grad_in, nxt))
        self._run(ops)
        io = None
        if recv_fwd:
            npos, ncu = hdr[7], hdr[6]
            io = StageIO(hidden_in, meta_in[:npos], meta_in[npos:npos + ncu] if ncu else None,
                         batch=hdr[2], seq=hdr[3], max_seqlen=hdr[4], max_position=hdr[5])
        return io, grad_in
