"""Mixed-precision optimizer on flat buffers with ZeRO-0/1/2 sharding over the DP group.

What the reference obtains from DeepSpeed (``BF16_Optimizer`` / ZeRO stage 0-2 wrapped
around apex FusedAdam: llm/utils/model/optimizer_helper.py:70-98,
llm/runners/base_llm_runner.py:194-213) re-designed around three flat buffers:

* ``param_buf``  — every trainable parameter of this rank re-homed into one contiguous
  buffer in the compute dtype (bf16 / fp16 / fp32); module parameters become views.
* ``grad_buf``   — fp32, same layout; each parameter gets ``main_grad`` (a view) that the
  wgrad GEMM / norm kernels accumulate into directly across micro-batches.
* ``master / m / v`` — fp32, only this DP rank's shard when ``stage >= 1``.

Stage 2 partitions the gradients as well (DeepSpeed ZeRO-2 with ``overlap_comm``, ``reduce_scatter``,
``contiguous_gradients``: configs/huggingface/template.yaml:13-21, scripts/ds_zero2_no_offload.json:11-19 of the
reference): there is no full ``grad_buf``.  Parameter gradients arrive through autograd hooks in the compute
dtype, are packed into a bucket (a few hundred MB, taken from a small pool), and a full bucket is reduced to the
owners of its ranges on a side stream while backward carries on; the owner adds its part into ``grad_acc``, its
fp32 shard, which is all that survives a micro-batch.  bf16 on the wire, fp32 accumulation over micro-batches.

One step = [TP all-reduce of sequence-parallel replicated grads] → DP reduce-scatter
(stage ≥ 1) or all-reduce (stage 0) of ``grad_buf`` → squared-norm partials → one world
all-reduce → clip coefficient kept on the device → fused Adam over the shard (writes the
low-precision shard of ``param_buf``) → DP all-gather of ``param_buf``.  No step of this
needs a host synchronisation except the optional fp16 overflow check.

Buffer order: [TP-sharded, decay][TP-sharded, no-decay][replicated, decay][replicated,
no-decay][replicated under sequence parallelism], so weight decay, norm de-duplication and
the TP gradient all-reduce each act on one contiguous range.
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist

from .. import ops
from ..parallel.grid import get_grid
from ..utils.log import default_logger as logger

_ALIGN = 8  # elements; keeps every shard boundary 16-byte aligned in bf16


def _no_decay(name, p):
    return name.endswith(".bias") or p.dim() == 1 or getattr(p, "no_weight_decay", False)


class DynamicLossScaler:
    """fp16 loss scaling (``optimizer.cur_scale`` in the reference's logger hook)."""

    def __init__(self, init_scale=2.0 ** 16, growth_interval=1000, factor=2.0, min_scale=1.0, hysteresis=2):
        self.cur_scale, self.growth_interval, self.factor = float(init_scale), growth_interval, factor
        self.min_scale, self.hysteresis, self._hyst, self._good = min_scale, hysteresis, hysteresis, 0

    def update(self, overflow: bool):
        if overflow:
            self._hyst -= 1
            if self._hyst <= 0:
                self.cur_scale = max(self.cur_scale / self.factor, self.min_scale)
            self._good = 0
        else:
            self._good += 1
            if self._good % self.growth_interval == 0:
                self.cur_scale *= self.factor
                self._hyst = self.hysteresis

    def state_dict(self):
        return {"cur_scale": self.cur_scale, "good": self._good, "hyst": self._hyst}

    def load_state_dict(self, s):
        self.cur_scale, self._good, self._hyst = s["cur_scale"], s["good"], s["hyst"]


class _NullCtx:
    def __enter__(self): return self
    def __exit__(self, *a): return False


class ZeroOptimizer:
    def __init__(self, named_params: Iterable, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 adamw=True, stage=1, grad_clip=0.0, fp16=False, bias_correction=True, loss_scale_cfg=None,
                 nan_policy="count", bucket_numel=1 << 27, max_buckets_in_flight=3):
        g = get_grid()
        self.grid = g
        self.stage = stage
        # ZeRO-2: gradients are partitioned too (only with a DP group to partition over)
        self.partitioned = stage >= 2 and g.dp > 1
        self.bucket_numel, self.max_buckets_in_flight = int(bucket_numel), int(max_buckets_in_flight)
        self.dp, self.dp_rank, self.dp_group = g.dp, g.dp_rank, g.dp_group
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.param_groups = [dict(self.defaults, name="all")]   # lr schedulers poke param_groups[i]['lr']
        self.adamw, self.grad_clip, self.bias_correction = adamw, grad_clip, bias_correction
        self.step_count = 0
        self.nan_policy = nan_policy
        self.skipped_steps = 0
        self.scaler = DynamicLossScaler(**(loss_scale_cfg or {})) if fp16 else None
        self._global_grad_norm = None

        named = [(n, p) for n, p in named_params if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        self.dtype = named[0][1].dtype
        self.device = named[0][1].device

        def klass(n, p):
            sharded = bool(getattr(p, "tensor_model_parallel", False))
            sp = bool(getattr(p, "sequence_parallel", False)) or bool(getattr(p, "tp_reduce_grad", False))
            if sp:
                return 4
            return (0 if sharded else 2) + (1 if _no_decay(n, p) else 0)

        order = sorted(range(len(named)), key=lambda i: (klass(*named[i]), i))
        self.names = [named[i][0] for i in order]
        self.params = [named[i][1] for i in order]
        klasses = [klass(named[i][0], named[i][1]) for i in order]
        self.offsets, off = [], 0
        bounds = {}
        for k, p in zip(klasses, self.params):
            bounds.setdefault(k, off)
            self.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.used = off
        # class range starts (monotone); missing classes collapse to the next start
        starts = []
        nxt = off
        for k in (4, 3, 2, 1, 0):
            nxt = bounds.get(k, nxt)
            starts.append(nxt)
        self.start_sp, self.start_rep_nd, self.start_rep, self.start_shard_nd, _ = starts
        chunk = _ALIGN * self.dp
        self.total = (off + chunk - 1) // chunk * chunk
        self.shard_size = self.total // self.dp if self.stage >= 1 else self.total
        self.shard_lo = self.dp_rank * self.shard_size if self.stage >= 1 else 0
        self.shard_hi = self.shard_lo + self.shard_size

        self.fused = False
        self.param_buf = self.grad_buf = None
        if self._want_fused():
            self._alloc_symmetric()
        if self.param_buf is None:
            self.param_buf = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        if self.grad_buf is None and not self.partitioned:
            self.grad_buf = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        for p, o in zip(self.params, self.offsets):
            view = self.param_buf[o:o + p.numel()].view_as(p)
            view.copy_(p.data)
            p.data = view
            if not self.partitioned:
                p.main_grad = self.grad_buf[o:o + p.numel()].view_as(p)
        if self.partitioned:
            self._init_partitioned_grads()
        self.master = self.param_buf[self.shard_lo:self.shard_hi].to(torch.float32, copy=True)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self._clip_coef = torch.ones(1, dtype=torch.float32, device=self.device)

    # ---- fused data-parallel path: buffers in symmetric memory, collectives issued by the kernels -------
    def _want_fused(self):
        import os
        return (self.dp > 1 and self.stage >= 1 and self.device.type == "cuda" and self.dtype == torch.bfloat16
                and ops.get_backend() == "b200" and os.environ.get("EASYLLM_ZERO_FUSED", "1") != "0"
                and dist.get_backend(self.dp_group) == "nccl" and self.dp <= 16)

    def _alloc_symmetric(self):
        """Flat gradient / parameter buffers every DP rank can address (NVLink peer pointers)."""
        try:
            import torch.distributed._symmetric_memory as symm_mem
            name = self.dp_group.group_name
            try:
                symm_mem.enable_symm_mem_for_group(name)
            except Exception:
                pass
            # ZeRO-2 keeps no full gradient buffer: only the parameter all-gather runs over symmetric memory
            gbuf = None if self.partitioned else symm_mem.empty(self.total, dtype=torch.float32, device=self.device)
            pbuf = symm_mem.empty(self.total, dtype=self.dtype, device=self.device)
            pbuf.zero_()
            gh = None
            if gbuf is not None:
                gbuf.zero_()
                gh = symm_mem.rendezvous(gbuf, group=name)
            ph = symm_mem.rendezvous(pbuf, group=name)
            torch.cuda.synchronize()
            dist.barrier(group=self.dp_group)
            self._grad_ptrs = [int(x) for x in gh.buffer_ptrs] if gh is not None else None
            self._param_ptrs = [int(x) for x in ph.buffer_ptrs]
            self._symm_handles = (gh, ph)
            self.grad_buf, self.param_buf = gbuf, pbuf
            self._sumsq2 = torch.zeros(2, dtype=torch.float32, device=self.device)
            self._dp_token = torch.zeros(1, dtype=torch.float32, device=self.device)
            self._have_sumsq2 = False
            self.fused = True
            logger.info(f"ZeRO-{self.stage}: fused " + ("" if self.partitioned else "reduce-scatter / ")
                        + f"Adam+all-gather kernels over {self.dp} ranks "
                        f"({self.total * (2 if self.partitioned else 6) / 2**30:.1f} GiB symmetric memory)")
        except Exception as e:   # no symmetric memory on this system: NCCL collectives instead
            logger.warning(f"ZeRO fused path unavailable ({type(e).__name__}: {e}); using NCCL collectives")
            self.fused = False
            self.param_buf = self.grad_buf = None

    def _dp_fence(self):
        """Stream-ordered rendezvous of the DP group: every rank's earlier kernels finished before any rank's
        later kernels start (a one-element all-reduce; no host synchronisation)."""
        dist.all_reduce(self._dp_token, group=self.dp_group)

    # ---- gradient plumbing --------------------------------------------------------------
    @property
    def cur_scale(self):
        return self.scaler.cur_scale if self.scaler else 1.0

    # ---- ZeRO-2: bucketed, overlapped reduction of partitioned gradients ------------------------------------
    def _init_partitioned_grads(self):
        """Buckets over the flat index space (whole parameters, at least ``bucket_numel`` elements each), the
        ranges of every bucket each DP rank owns, and an autograd hook per parameter."""
        self.grad_acc = torch.zeros(self.shard_size, dtype=torch.float32, device=self.device)
        self._buckets = []
        cur = None
        for i, (p, o) in enumerate(zip(self.params, self.offsets)):
            if cur is None:
                cur = {"lo": o, "params": [], "hi": o}
            cur["params"].append(i)
            cur["hi"] = o + (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
            if cur["hi"] - cur["lo"] >= self.bucket_numel:
                self._buckets.append(cur)
                cur = None
        if cur is not None:
            self._buckets.append(cur)
        self._bucket_of = {}
        for bi, b in enumerate(self._buckets):
            b["segments"] = []
            for r in range(self.dp):
                lo, hi = max(b["lo"], r * self.shard_size), min(b["hi"], (r + 1) * self.shard_size)
                if hi > lo:
                    b["segments"].append((r, lo, hi))
            # gradients of TP-replicated parameters under sequence parallelism are summed over TP first
            b["tp_range"] = (max(b["lo"], self.start_sp), min(b["hi"], self.used))
            b.update(buf=None, got=set(), fired=False)
            for i in b["params"]:
                self._bucket_of[id(self.params[i])] = (bi, i)
        self._bucket_cap = max(b["hi"] - b["lo"] for b in self._buckets)
        self._free_bufs, self._inflight = [], []
        self._n_bufs = 0
        self._dp_ranks = dist.get_process_group_ranks(self.dp_group) if dist.is_initialized() else [0]
        self._comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._hooks = [p.register_post_accumulate_grad_hook(self._grad_hook) for p in self.params]
        logger.info(f"ZeRO-2: gradients partitioned over {self.dp} ranks, {len(self._buckets)} buckets of up to "
                    f"{self._bucket_cap * self.param_buf.element_size() / 2**20:.0f} MiB")

    def _acquire_bucket_buffer(self):
        if self._free_bufs:
            return self._free_bufs.pop()
        if self._n_bufs >= self.max_buckets_in_flight and self._inflight:
            buf, done = self._inflight.pop(0)          # the oldest reduction: the compute stream waits for it
            if done is not None:
                torch.cuda.current_stream().wait_event(done)
            return buf
        self._n_bufs += 1
        return torch.empty(self._bucket_cap, dtype=self.dtype, device=self.device)

    def _grad_hook(self, p):
        """Runs inside backward as soon as ``p.grad`` is final for this micro-batch: pack it into its bucket,
        free it, and reduce the bucket once every one of its parameters has arrived."""
        bi, i = self._bucket_of[id(p)]
        b = self._buckets[bi]
        if b["fired"]:
            raise RuntimeError(f"gradient of {self.names[i]} arrived after its bucket was reduced; a parameter "
                               "that receives gradients twice per backward needs ZeRO stage <= 1")
        if b["buf"] is None:
            b["buf"] = self._acquire_bucket_buffer()
        o = self.offsets[i] - b["lo"]
        view = b["buf"][o:o + p.numel()].view_as(p)
        if i in b["got"]:
            view.add_(p.grad)
        else:
            view.copy_(p.grad)
            b["got"].add(i)
        p.grad = None
        if len(b["got"]) == len(b["params"]):
            self._reduce_bucket(b)

    def _reduce_bucket(self, b):
        """Reduce every range of the bucket to the rank that owns it (its part of the ZeRO shard) and let the owner
        add it into ``grad_acc``; on a GPU this runs on a side stream, overlapped with the rest of backward."""
        b["fired"] = True
        if b["buf"] is None:
            b["buf"] = self._acquire_bucket_buffer()
        buf = b["buf"]
        for i in b["params"]:                          # parameters without a gradient this time count as zero
            if i not in b["got"]:
                o = self.offsets[i] - b["lo"]
                buf[o:o + self.params[i].numel()].zero_()
        g = self.grid
        tlo, thi = b["tp_range"]
        if g.tp > 1 and thi > tlo:
            dist.all_reduce(buf[tlo - b["lo"]:thi - b["lo"]], group=g.tp_group)
        cuda = self._comm_stream is not None
        if cuda:
            ready = torch.cuda.Event()
            ready.record()
            self._comm_stream.wait_event(ready)
        ctx = torch.cuda.stream(self._comm_stream) if cuda else _NullCtx()
        with ctx:
            for owner, lo, hi in b["segments"]:
                seg = buf[lo - b["lo"]:hi - b["lo"]]
                dist.reduce(seg, dst=self._dp_ranks[owner], group=self.dp_group)
                if owner == self.dp_rank:
                    dst = self.grad_acc[lo - self.shard_lo:hi - self.shard_lo]
                    if cuda and seg.dtype == torch.bfloat16 and ops.get_backend() == "b200":
                        from ..ops import cuda as cu
                        cu.accum_bf16_to_f32(seg, dst)
                    else:
                        dst.add_(seg.float())
            done = None
            if cuda:
                done = torch.cuda.Event()
                done.record(self._comm_stream)
        self._inflight.append((buf, done))
        b["buf"] = None

    def _flush_buckets(self):
        """End of a micro-batch's backward: reduce what the hooks have not (the same sequence of collectives on
        every rank, whatever gradients were produced), then make the compute stream wait for the reductions."""
        for b in self._buckets:
            if not b["fired"]:
                self._reduce_bucket(b)
        for buf, done in self._inflight:
            if done is not None:
                torch.cuda.current_stream().wait_event(done)
            self._free_bufs.append(buf)
        self._inflight = []
        for b in self._buckets:
            b.update(buf=None, got=set(), fired=False)

    def accumulate_grads(self):
        """Fold autograd ``.grad`` tensors (reference / CPU path) into ``main_grad``; with partitioned gradients
        (ZeRO-2) finish this micro-batch's bucket reductions instead."""
        if self.partitioned:
            self._flush_buckets()
            return
        for p in self.params:
            if p.grad is not None:
                if p.grad.is_cuda and p.grad.dtype == torch.bfloat16 and ops.get_backend() == "b200" \
                        and p.grad.is_contiguous():
                    from ..ops import cuda
                    cuda.accum_bf16_to_f32(p.grad, p.main_grad)
                else:
                    p.main_grad.add_(p.grad.float())
                p.grad = None

    def zero_grad(self):
        (self.grad_acc if self.partitioned else self.grad_buf).zero_()
        for p in self.params:
            p.grad = None

    def _segment_sumsq(self, lo, hi):
        lo, hi = max(lo, self.shard_lo), min(hi, self.shard_hi)
        if hi <= lo:
            return torch.zeros(1, dtype=torch.float32, device=self.device)
        return ops.sumsq(self._grad_shard()[lo - self.shard_lo:hi - self.shard_lo])

    def _grad_shard(self):
        if self.partitioned:
            return self.grad_acc
        return self.grad_buf[self.shard_lo:self.shard_hi]

    def reduce_gradients(self):
        g = self.grid
        if self.partitioned:
            return                                    # reduced bucket by bucket during the backward passes
        if g.tp > 1 and self.start_sp < self.used:
            dist.all_reduce(self.grad_buf[self.start_sp:self.used], group=g.tp_group)
        if self.fused and not self.partitioned:
            from ctypes import c_int, c_longlong, c_void_p
            from ..ops import cuda as cu
            self._dp_fence()                      # every rank's backward (and TP reduce) is complete
            self._sumsq2.zero_()
            arr = (c_void_p * self.dp)(*self._grad_ptrs)
            rc = cu.lib().ell_zero_reduce_scatter(arr, c_int(self.dp), c_int(self.dp_rank), c_longlong(self.shard_lo),
                                                  c_longlong(self.shard_size), c_longlong(self.start_rep),
                                                  cu._p(self._sumsq2), cu._stream())
            cu._check(rc, "zero_reduce_scatter")
            cu.LAUNCHES += 1
            self._have_sumsq2 = True
            return
        if self.dp > 1:
            self.grad_buf.div_(self.dp)
            if self.stage >= 1 and dist.get_backend(self.dp_group) != "gloo":
                dist.reduce_scatter_tensor(self._grad_shard(), self.grad_buf, group=self.dp_group)
            else:
                dist.all_reduce(self.grad_buf, group=self.dp_group)

    def compute_grad_norm(self):
        """Global L2 norm of the (unscaled) gradients as a device tensor, every parameter
        counted once: replicated ranges only on tp_rank 0, ZeRO shards summed over DP."""
        g = self.grid
        if self.fused and self._have_sumsq2:      # produced by the reduce-scatter kernel in the same pass
            sq = self._sumsq2[0:1].clone()
            if g.tp_rank == 0:
                sq = sq + self._sumsq2[1:2]
            self._have_sumsq2 = False
        else:
            sq = self._segment_sumsq(0, self.start_rep)
            if g.tp_rank == 0:
                sq = sq + self._segment_sumsq(self.start_rep, self.used)
        if dist.is_initialized() and g.world > 1:
            if self.stage >= 1:
                dist.all_reduce(sq)                       # dp shards × tp × pp
            elif g.mp_group is not None and g.tp * g.pp > 1:
                dist.all_reduce(sq, group=g.mp_group)
        # ZeRO-2 accumulates the SUM over the DP ranks; the mean's 1/dp is folded in here and into the update
        norm = sq.sqrt() / (self.cur_scale * self._dp_sum_factor())
        self._global_grad_norm = norm
        return norm

    def _dp_sum_factor(self):
        return float(self.dp) if self.partitioned else 1.0

    def get_global_grad_norm(self):
        return None if self._global_grad_norm is None else float(self._global_grad_norm)

    # ---- the step ---------------------------------------------------------------------------
    def step(self):
        """reduce → norm/clip → Adam on the shard → all-gather.  Returns False if skipped."""
        self.reduce_gradients()
        norm = self.compute_grad_norm()
        finite_needed = self.scaler is not None or self.nan_policy in ("skip", "abort")
        if finite_needed:
            ok = bool(torch.isfinite(norm))
            if self.scaler is not None:
                self.scaler.update(not ok)
            if not ok:
                if self.nan_policy == "abort":
                    raise FloatingPointError("non-finite gradient norm")
                self.skipped_steps += 1
                self.zero_grad()
                return False
        if self.grad_clip and self.grad_clip > 0:
            torch.clamp(self.grad_clip / (norm + 1e-6), max=1.0, out=self._clip_coef)
        else:
            self._clip_coef.fill_(1.0)
        self.step_count += 1
        pg = self.param_groups[0]
        lr, betas, eps, wd = pg["lr"], pg["betas"], pg["eps"], pg["weight_decay"]
        inv_scale = 1.0 / (self.cur_scale * self._dp_sum_factor())
        if self.fused and self.partitioned:
            self._dp_fence()                      # every rank is done with the old parameters
        # weight decay applies to [0, start_shard_nd) ∪ [start_rep, start_rep_nd)
        cuts = [0, self.start_shard_nd, self.start_rep, self.start_rep_nd, self.total]
        wds = [wd, 0.0, wd, 0.0]
        lowp = self.param_buf[self.shard_lo:self.shard_hi]
        gsh = self._grad_shard()
        for (a, b), w in zip(zip(cuts[:-1], cuts[1:]), wds):
            lo, hi = max(a, self.shard_lo) - self.shard_lo, min(b, self.shard_hi) - self.shard_lo
            if hi <= lo:
                continue
            if self.fused:
                self._fused_adam_allgather(lo, hi, lr, betas, eps, w, inv_scale)
                continue
            ops.fused_adam_(self.master[lo:hi], gsh[lo:hi], self.exp_avg[lo:hi], self.exp_avg_sq[lo:hi], lowp[lo:hi],
                            lr, betas, eps, w, self.step_count, self.adamw, inv_scale, self._clip_coef,
                            self.bias_correction)
        if self.fused:
            self._dp_fence()                      # peers' parameter stores have landed; their gradient reads are done
        elif self.stage >= 1 and self.dp > 1:
            if dist.get_backend(self.dp_group) == "gloo":
                parts = [torch.empty_like(lowp) for _ in range(self.dp)]
                dist.all_gather(parts, lowp.contiguous(), group=self.dp_group)
                self.param_buf.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(self.param_buf, lowp, group=self.dp_group)
        self.zero_grad()
        return True

    def _fused_adam_allgather(self, lo, hi, lr, betas, eps, wd, inv_scale):
        """Adam on master[lo:hi] with the bf16 result stored into every DP rank's parameter buffer."""
        from ctypes import c_float, c_int, c_longlong, c_void_p
        from ..ops import cuda as cu
        c1 = 1.0 - betas[0] ** self.step_count if self.bias_correction else 1.0
        c2 = 1.0 - betas[1] ** self.step_count if self.bias_correction else 1.0
        arr = (c_void_p * self.dp)(*self._param_ptrs)
        gsh = self._grad_shard()
        rc = cu.lib().ell_zero_adam_allgather(
            arr, c_int(self.dp), c_int(self.dp_rank), c_longlong(self.shard_lo + lo), c_longlong(hi - lo),
            cu._p(self.master[lo:hi]), cu._p(gsh[lo:hi]), cu._p(self.exp_avg[lo:hi]), cu._p(self.exp_avg_sq[lo:hi]),
            c_float(lr), c_float(betas[0]), c_float(betas[1]), c_float(eps), c_float(wd), c_float(c1), c_float(c2),
            c_float(inv_scale), c_int(1 if self.adamw else 0), cu._p(self._clip_coef), cu._stream())
        cu._check(rc, "zero_adam_allgather")
        cu.LAUNCHES += 1

    def refresh_fp32_params(self):
        """Re-derive the fp32 master shard from the (just loaded) low-precision parameters."""
        self.master.copy_(self.param_buf[self.shard_lo:self.shard_hi].float())

    # ---- checkpoint ---------------------------------------------------------------------------
    def state_dict(self):
        return {"step": self.step_count, "stage": self.stage, "dp": self.dp, "dp_rank": self.dp_rank,
                "total": self.total, "used": self.used, "shard_lo": self.shard_lo, "shard_hi": self.shard_hi,
                "names": self.names, "offsets": self.offsets, "numels": [p.numel() for p in self.params],
                "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(), "exp_avg_sq": self.exp_avg_sq.cpu(),
                "param_groups": [{k: v for k, v in pg.items()} for pg in self.param_groups],
                "scaler": self.scaler.state_dict() if self.scaler else None, "skipped_steps": self.skipped_steps}

    def load_state_dict(self, sd, load_param_groups=True):
        if sd["total"] != self.total or sd["shard_lo"] != self.shard_lo or sd["shard_hi"] != self.shard_hi:
            raise ValueError("optimizer shard layout differs; use load_resharded() with all shards")
        self.step_count = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        if load_param_groups:
            for pg, s in zip(self.param_groups, sd["param_groups"]):
                pg.update(s)
        if self.scaler and sd.get("scaler"):
            self.scaler.load_state_dict(sd["scaler"])
        self.skipped_steps = sd.get("skipped_steps", 0)

    def load_resharded(self, shards: List[dict]):
        """Load from the optimizer shards of a run with a different DP size: the flat fp32
        state is re-assembled by parameter name, then re-sliced for this rank."""
        full = {}
        for key in ("master", "exp_avg", "exp_avg_sq"):
            cat = torch.cat([s[key] for s in sorted(shards, key=lambda s: s["shard_lo"])])
            full[key] = cat
        src = shards[0]
        by_name = {n: (o, k) for n, o, k in zip(src["names"], src["offsets"], src["numels"])}
        for key, dst in (("master", self.master), ("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
            flat = torch.zeros(self.total, dtype=torch.float32)
            for n, o, p in zip(self.names, self.offsets, self.params):
                so, k = by_name[n]
                flat[o:o + k] = full[key][so:so + k]
            dst.copy_(flat[self.shard_lo:self.shard_hi])
        self.step_count = src["step"]
