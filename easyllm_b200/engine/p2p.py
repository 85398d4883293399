"""Pipeline-stage point-to-point exchange of activations and gradients.

Stays on ``torch.distributed`` p2p (NCCL on GPUs, gloo on CPU) by design: a stage boundary moves one
``[T/tp, h]`` tensor per micro-batch.  What this module adds is the overlap under the 1F1B schedule:

* activations (stage s → s+1) and gradients (s+1 → s) travel on two separate process groups, i.e. two NCCL
  communicators with their own streams, so neither direction queues behind the other;
* every transfer is asynchronous: a send only keeps its tensors alive until it has completed, and the receive of the
  NEXT micro-batch is posted right after the send of the current one, so it lands while the stage computes;
* the shape header of a forward message goes through a CPU (gloo) group as a host tensor: with ``dynamic=True``
  (micro-batches of different token counts: ``runtime.dynamic`` of the reference,
  llm/runners/base_llm_runner.py:240-242) reading it costs no device synchronisation; otherwise the first header is
  cached and no further header is sent.

One forward message = header int64[8] (host) + hidden ``[T_local, h]`` + int32 meta ``[T + n_cu]`` (position ids,
then cu_seqlens).  Backward messages are the hidden gradient.  Within one direction messages are FIFO.
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


class _Pending:
    """An in-flight transfer: its work handles and the tensors they read or fill."""

    def __init__(self, works, tensors):
        self.works, self.tensors = works, tensors

    def wait(self):
        for w in self.works:
            w.wait()
        self.works = []


class StageLink:
    def __init__(self, dtype, dynamic=True):
        self.g = get_grid()
        self.dtype = dtype
        self._dynamic = dynamic
        self._cached_hdr = None       # receiver side (static shapes)
        self._sent_hdr = False        # sender side (static shapes)
        self._sends = []              # sends not yet known to be complete
        self._recv_fwd = None         # (header work | None, header tensor | None, payload _Pending | None)
        self._recv_bwd = None

    @property
    def dynamic(self):
        return self._dynamic

    @dynamic.setter
    def dynamic(self, value):
        """Every stage switches together (the engine passes the same flag on all of them); a switch forgets the
        cached header, so the first message of a static phase carries one again."""
        if bool(value) != self._dynamic:
            self._dynamic = bool(value)
            self._cached_hdr, self._sent_hdr = None, False

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

    def _reap_sends(self):
        self._sends = [p for p in self._sends if not all(w.is_completed() for w in p.works)]

    # ---- forward direction: activations ------------------------------------------------------------
    def send_fwd(self, io: StageIO):
        """Start sending this stage's output to the next stage; returns at once."""
        g = self.g
        nxt = g.next_stage_rank()
        works, keep = [], []
        if self.dynamic or not self._sent_hdr:
            hdr = self._header_of(io)
            works.append(dist.isend(hdr, nxt, group=g.pp_host_group))
            keep.append(hdr)
            self._sent_hdr = True
        hidden = io.hidden.detach().contiguous()
        meta = self._meta_of(io).to(_dev())
        works.append(dist.isend(hidden, nxt, group=g.pp_fwd_group))
        works.append(dist.isend(meta, nxt, group=g.pp_fwd_group))
        keep += [hidden, meta]
        self._reap_sends()
        self._sends.append(_Pending(works, keep))

    def _post_fwd_payload(self, hdr):
        g = self.g
        prv, dev = g.prev_stage_rank(), _dev()
        hidden = torch.empty(hdr[0], hdr[1], dtype=self.dtype, device=dev)
        meta = torch.empty(hdr[7] + hdr[6], dtype=torch.int32, device=dev)
        works = [dist.irecv(hidden, prv, group=g.pp_fwd_group), dist.irecv(meta, prv, group=g.pp_fwd_group)]
        return _Pending(works, (hidden, meta, hdr))

    def post_recv_fwd(self):
        """Start receiving the next forward input.  With static shapes (header cached) the payload receive is posted
        right away; otherwise the header receive is, and the payload follows once the header is here."""
        if self._recv_fwd is not None:
            return
        g = self.g
        if not self.dynamic and self._cached_hdr is not None:
            self._recv_fwd = (None, None, self._post_fwd_payload(self._cached_hdr))
            return
        hdr = torch.empty(_HDR, dtype=torch.int64)
        self._recv_fwd = (dist.irecv(hdr, g.prev_stage_rank(), group=g.pp_host_group), hdr, None)

    def wait_recv_fwd(self) -> StageIO:
        if self._recv_fwd is None:
            self.post_recv_fwd()
        hwork, hdr_t, payload = self._recv_fwd
        self._recv_fwd = None
        if payload is None:
            hwork.wait()                               # a host tensor on the CPU group: no device synchronisation
            hdr = hdr_t.tolist()
            self._cached_hdr = hdr
            payload = self._post_fwd_payload(hdr)
        payload.wait()
        hidden, meta, hdr = payload.tensors
        npos, ncu = hdr[7], hdr[6]
        return StageIO(hidden, meta[:npos], meta[npos:npos + ncu] if ncu else None,
                       batch=hdr[2], seq=hdr[3], max_seqlen=hdr[4], max_position=hdr[5])

    # ---- backward direction: gradients ---------------------------------------------------------------
    def send_bwd(self, grad: torch.Tensor):
        g = self.g
        t = grad.contiguous()
        self._reap_sends()
        self._sends.append(_Pending([dist.isend(t, g.prev_stage_rank(), group=g.pp_bwd_group)], [t]))

    def post_recv_bwd(self, like: torch.Tensor):
        """Start receiving the gradient of an output this stage sent earlier (``like``: that output)."""
        if self._recv_bwd is not None:
            return
        g = self.g
        buf = torch.empty_like(like)
        self._recv_bwd = _Pending([dist.irecv(buf, g.next_stage_rank(), group=g.pp_bwd_group)], (buf,))

    def wait_recv_bwd(self, like: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self._recv_bwd is None:
            self.post_recv_bwd(like)
        p, self._recv_bwd = self._recv_bwd, None
        p.wait()
        return p.tensors[0]

    def flush(self):
        """Wait for every send issued so far (end of a batch: their tensors may be released)."""
        for p in self._sends:
            p.wait()
        self._sends = []
