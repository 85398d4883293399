"""Index samplers (llm/data/nlp_sampler.py:8-247).

* ``megatron_pretrain`` — sequential; every group of ``micro_batch · dp`` consecutive samples
  is split across DP ranks; resumes from ``consumed_samples``.
* ``megatron_pretrain_random`` — each DP rank owns one contiguous bucket, permuted per epoch
  with the epoch number as seed; resumes mid-epoch from ``consumed_samples``.
* ``dist`` / ``dist_test`` samplers + ``base`` batch sampler + ``InfiniteBatchSampler`` for the
  HF-style runner (epoch-seeded permutation, padded to a multiple of the DP size; the test
  variant does not pad, so no sample is evaluated twice).
"""
from __future__ import annotations

import math

import torch
from torch.utils.data.sampler import BatchSampler, Sampler

from ..config.registry import BATCH_SAMPLER_REGISTRY, SAMPLER_REGISTRY


def _check(total, mbs, dp_rank, dp_size):
    if total <= 0:
        raise ValueError(f"no sample to consume: {total}")
    if mbs <= 0 or dp_size <= 0 or not 0 <= dp_rank < dp_size:
        raise ValueError("bad micro_batch_size / data parallel rank / size")


@BATCH_SAMPLER_REGISTRY.register("megatron_pretrain")
class MegatronPretrainingSampler:
    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank, data_parallel_size,
                 drop_last=True):
        _check(total_samples, micro_batch_size, data_parallel_rank, data_parallel_size)
        if consumed_samples >= total_samples:
            raise ValueError(f"no samples left to consume: {consumed_samples}, {total_samples}")
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size, self.data_parallel_rank = micro_batch_size, data_parallel_rank
        self.group = micro_batch_size * data_parallel_size
        self.drop_last = drop_last

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        lo = self.data_parallel_rank * self.micro_batch_size
        for start in range(self.consumed_samples, self.total_samples, self.group):
            end = min(start + self.group, self.total_samples)
            if end - start < self.group and self.drop_last:
                return
            yield list(range(start, end))[lo:lo + self.micro_batch_size]


@BATCH_SAMPLER_REGISTRY.register("megatron_pretrain_random")
class MegatronPretrainingRandomSampler:
    def __init__(self, total_samples, consumed_samples, micro_batch_size, data_parallel_rank, data_parallel_size):
        _check(total_samples, micro_batch_size, data_parallel_rank, data_parallel_size)
        self.total_samples, self.consumed_samples = total_samples, consumed_samples
        self.micro_batch_size = micro_batch_size
        self.data_parallel_rank, self.data_parallel_size = data_parallel_rank, data_parallel_size
        self.group = micro_batch_size * data_parallel_size
        self.last_batch_size = total_samples % self.group

    def __len__(self):
        return self.total_samples

    def __iter__(self):
        active = self.total_samples - self.last_batch_size
        self.epoch = self.consumed_samples // active
        in_epoch = self.consumed_samples % active
        if in_epoch % self.group:
            raise ValueError("consumed_samples is not a multiple of micro_batch_size × data_parallel_size")
        bucket = (self.total_samples // self.group) * self.micro_batch_size
        offset = in_epoch // self.data_parallel_size
        base = self.data_parallel_rank * bucket
        g = torch.Generator()
        g.manual_seed(self.epoch)
        order = torch.randperm(bucket, generator=g).tolist()[offset:]
        for i in range(0, len(order) - self.micro_batch_size + 1, self.micro_batch_size):
            self.consumed_samples += self.group
            yield [base + x for x in order[i:i + self.micro_batch_size]]


@SAMPLER_REGISTRY.register("dist_test")
class TestDistributedSampler(Sampler):
    __test__ = False

    def __init__(self, dataset_size=None, data_parallel_rank=0, data_parallel_size=1, total_samples=None):
        self.dataset_size = dataset_size if dataset_size is not None else total_samples
        self.num_replicas, self.rank, self.epoch = data_parallel_size, data_parallel_rank, 0
        self.num_samples = len(range(self.rank, self.dataset_size, self.num_replicas))

    def __iter__(self):
        return iter(range(self.rank, self.dataset_size, self.num_replicas))

    def __len__(self):
        return self.num_samples

    def set_epoch(self, epoch):
        self.epoch = epoch


@SAMPLER_REGISTRY.register("dist")
class DistributedSampler(Sampler):
    def __init__(self, dataset_size=None, data_parallel_rank=0, data_parallel_size=1, total_samples=None):
        self.dataset_size = dataset_size if dataset_size is not None else total_samples
        self.num_replicas, self.rank, self.epoch = data_parallel_size, data_parallel_rank, 0
        self.num_samples = int(math.ceil(self.dataset_size / self.num_replicas))
        self.total_size = self.num_samples * self.num_replicas
        self.consumed_samples = 0

    def __iter__(self):
        self.epoch = self.consumed_samples // self.total_size
        done = self.consumed_samples % self.total_size
        if done % self.num_replicas:
            self.consumed_samples -= done % self.num_replicas
            done -= done % self.num_replicas
        g = torch.Generator()
        g.manual_seed(self.epoch)
        idx = torch.randperm(self.dataset_size, generator=g).tolist()
        pad = self.total_size - len(idx)
        idx += (idx * math.ceil(pad / max(1, len(idx))))[:pad] if pad else []
        lo = self.num_samples * self.rank + done // self.num_replicas
        return iter(idx[lo:self.num_samples * (self.rank + 1)])

    def __len__(self):
        return self.num_samples

    def set_epoch(self, epoch):
        self.epoch = epoch

    def set_consumed_samples(self, consumed_samples):
        self.consumed_samples = consumed_samples


@BATCH_SAMPLER_REGISTRY.register("base")
class BaseBatchSampler(BatchSampler):
    def __init__(self, sampler, batch_size, drop_last=False):
        super().__init__(sampler, batch_size, drop_last)

    def set_consumed_samples(self, consumed_samples):
        self.sampler.set_consumed_samples(consumed_samples)


class InfiniteBatchSampler:
    """Cycles a batch sampler forever, tracking globally consumed samples for resume."""

    def __init__(self, batch_sampler, start_iter=0):
        self.batch_sampler = batch_sampler
        self.batch_size = batch_sampler.batch_size
        self.data_parallel_size = batch_sampler.sampler.num_replicas
        self.consumed_samples = 0

    def __iter__(self):
        while True:
            if hasattr(self.batch_sampler.sampler, "set_consumed_samples"):
                self.batch_sampler.sampler.set_consumed_samples(self.consumed_samples)
            for batch in self.batch_sampler:
                self.consumed_samples += len(batch) * self.data_parallel_size
                yield batch

    def __len__(self):
        return len(self.batch_sampler)

    def set_consumed_samples(self, consumed_samples):
        self.batch_sampler.sampler.set_consumed_samples(consumed_samples)
        self.consumed_samples = consumed_samples


def build_batch_sampler(cfg):
    kw = cfg.get("kwargs") or {}
    if cfg["type"] == "base" and "sampler" in kw:
        scfg = {"type": kw["sampler"]["type"], "kwargs": dict(kw["sampler"].get("kwargs") or {})}
        scfg["kwargs"].update(total_samples=kw["total_samples"], data_parallel_rank=kw["data_parallel_rank"],
                              data_parallel_size=kw["data_parallel_size"])
        sampler = SAMPLER_REGISTRY.build(scfg)
        return InfiniteBatchSampler(BaseBatchSampler(sampler, kw["micro_batch_size"]))
    return BATCH_SAMPLER_REGISTRY.build(cfg)
