"""Data loader, batch-pipe functions and the iterator builder.

Parity: llm/data/nlp_dataloader.py:216-320 (``base`` loader: seeded worker processes, batch
sampler + collator, ``get_epoch_size``), llm/data/nlp_batch_fn.py:7-284 (``json_batch_pipe``,
``flash_batch_pipe``, ``mini_rlhf_json_batch_pipe``, ``token_batch_pipe``) and
llm/data/build.py:14-48 (only TP rank 0 owns a loader; micro-batches are broadcast to the
TP group inside the batch function).

Batch functions return ``((tokens, position_ids, attention_mask[, cu_seqlens]), (labels,
loss_mask[, scores]))``.  The attention kernels are causal and segment-aware, so no dense
``[s, s]`` mask is built: ``attention_mask`` is ``None`` (causal) and a document reset
(``reset_attention_mask``) is expressed as ``cu_seqlens``; ``dense_mask=True`` restores the
dense boolean mask for debugging.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from ..config.registry import BATCH_COLLECTOR_REGISTRY, BATCH_FN_REGISTRY, DATALOADER_REGISTRY
from ..parallel.data import broadcast_data
from ..parallel.grid import get_grid
from . import collators as _c  # noqa: F401  (registers collators)
from .datasets import build_dataset
from .samplers import build_batch_sampler


def _seed_worker(base_seed):
    def init(worker_id):
        import random
        import numpy as np
        s = (base_seed + worker_id) % (2 ** 32)
        random.seed(s)
        np.random.seed(s)
        torch.manual_seed(s)
    return init


@DATALOADER_REGISTRY.register("base")
class BaseDataLoader(DataLoader):
    def __init__(self, dataset, batch_sampler=None, batch_collator=None, num_workers=0, pin_memory=False, seed=0,
                 prefetch_factor=None, persistent_workers=False, **kw):
        g = torch.Generator()
        g.manual_seed(seed)
        extra = {}
        if num_workers > 0:
            extra = dict(prefetch_factor=prefetch_factor or 2, persistent_workers=persistent_workers,
                         worker_init_fn=_seed_worker(seed))
        super().__init__(dataset, batch_sampler=batch_sampler, collate_fn=batch_collator, num_workers=num_workers,
                         pin_memory=pin_memory and torch.cuda.is_available(), generator=g, **extra)

    def get_epoch_size(self):
        bs = getattr(self.batch_sampler, "micro_batch_size", None) or getattr(self.batch_sampler, "batch_size", 1)
        return math.ceil(len(self.batch_sampler) / bs) if hasattr(self.batch_sampler, "__len__") else 0


def build_batch_collator(cfg, tokenizer):
    cfg = {"type": cfg["type"], "kwargs": dict(cfg.get("kwargs") or {})}
    cfg["kwargs"]["tokenizer"] = tokenizer
    return BATCH_COLLECTOR_REGISTRY.build(cfg)


def build_data_loader(cfg, dataset, batch_sampler, batch_collator):
    cfg = {"type": cfg.get("type", "base"), "kwargs": dict(cfg.get("kwargs") or {})}
    cfg["kwargs"].update(dataset=dataset, batch_sampler=batch_sampler, batch_collator=batch_collator)
    return DATALOADER_REGISTRY.build(cfg)


# ---- masks / positions --------------------------------------------------------------------------
def get_ltor_masks_and_position_ids(data, eod_token, reset_position_ids, reset_attention_mask, eod_mask_loss,
                                    prefix_indices=None, loss_on_targets_only=True, dense_mask=False):
    """Left-to-right loss mask, position ids and document boundaries.

    Returns ``(attention_mask | None, loss_mask, position_ids, cu_seqlens | None)``.  Documents
    end *after* an EOD token.  With ``dense_mask`` the boolean ``[b,1,s,s]`` mask (True = masked)
    of the reference is also built."""
    b, s = data.shape
    dev = data.device
    loss_mask = torch.ones(b, s, dtype=torch.float, device=dev)
    if eod_mask_loss:
        loss_mask[data == eod_token] = 0.0
    pos = torch.arange(s, dtype=torch.long, device=dev).unsqueeze(0).expand(b, s)
    cu = None
    need_docs = reset_position_ids or reset_attention_mask
    starts_all = []
    if need_docs:
        pos = pos.clone()
        for i in range(b):
            ends = (torch.nonzero(data[i] == eod_token).flatten() + 1).tolist()
            ends = [e for e in ends if e < s]
            starts = [0] + ends
            starts_all.append(starts)
            if reset_position_ids:
                for st in starts[1:]:
                    pos[i, st:] = torch.arange(s - st, device=dev)
        if reset_attention_mask:
            flat = [i * s + st for i, sts in enumerate(starts_all) for st in sts] + [b * s]
            cu = torch.tensor(flat, dtype=torch.int32, device=dev)
    if prefix_indices is not None and loss_on_targets_only:
        for i in range(b):
            p = prefix_indices[i]
            if isinstance(p, int):
                loss_mask[i, :p - 1] = 0.0
            else:
                prev = 0
                for j, pj in enumerate(p):
                    loss_mask[i, prev:pj - 1] = 0.0
                    prev = starts_all[i][j + 1] if starts_all and j + 1 < len(starts_all[i]) else s
    mask = None
    if dense_mask:
        nb = b if (reset_attention_mask or prefix_indices is not None) else 1
        m = torch.tril(torch.ones(nb, s, s, device=dev)).view(nb, 1, s, s)
        if reset_attention_mask:
            for i in range(b):
                for st in starts_all[i][1:]:
                    m[i, 0, st:, :st] = 0
        mask = m < 0.5
    return mask, loss_mask, pos, cu


def get_peft_attention_mask(tokens, eod_token):
    """HF-style combined causal + padding mask (True = masked), ``[b,1,s,s]``."""
    b, s = tokens.shape
    causal = torch.triu(torch.ones(s, s, dtype=torch.bool, device=tokens.device), diagonal=1)
    pad = (tokens == eod_token)[:, None, None, :].expand(b, 1, s, s)
    return pad | causal[None, None]


class _PipeBase:
    def __init__(self, tokenizer):
        self.tokenizer = tokenizer
        self.pad_token_id = len(tokenizer) - 1


@BATCH_FN_REGISTRY.register("json_batch_pipe")
class JsonBatchFunction(_PipeBase):
    def __init__(self, tokenizer, reset_position_ids=False, reset_attention_mask=False, eod_mask_loss=True,
                 prefix_indices=None, loss_on_targets_only=True, hf_atten_mask=False, dense_mask=False):
        super().__init__(tokenizer)
        self.a = (reset_position_ids, reset_attention_mask, eod_mask_loss, prefix_indices, loss_on_targets_only)
        self.hf_atten_mask, self.dense_mask = hf_atten_mask, dense_mask

    def __call__(self, data):
        d = broadcast_data(["labels", "input_ids"], data, torch.int64)
        labels, tokens = d["labels"].long(), d["input_ids"].long()
        mask, loss_mask, pos, cu = get_ltor_masks_and_position_ids(tokens, self.pad_token_id, *self.a,
                                                                   dense_mask=self.dense_mask)
        if self.hf_atten_mask and self.dense_mask:
            mask = get_peft_attention_mask(tokens, self.pad_token_id)
        inputs = (tokens, pos, mask) if cu is None else (tokens, pos, mask, cu)
        return inputs, (labels, loss_mask)


@BATCH_FN_REGISTRY.register("flash_batch_pipe")
class FlashBatchFunction(_PipeBase):
    def __init__(self, tokenizer, eod_mask_loss=True, pretrain=False):
        super().__init__(tokenizer)
        self.eod_mask_loss, self.pretrain = eod_mask_loss, pretrain

    def __call__(self, data):
        keys = ["labels", "input_ids"] + (["cu_seqlens", "position_ids"] if self.pretrain else [])
        d = broadcast_data(keys, data, torch.int64)
        labels, tokens = d["labels"].long(), d["input_ids"].long()
        mask = tokens.ne(self.pad_token_id)
        if not self.pretrain:
            pos = torch.arange(tokens.shape[1], dtype=torch.long, device=tokens.device).unsqueeze(0).expand_as(tokens)
            return (tokens, pos, mask), (labels, mask.clone())
        return (tokens, d["position_ids"], mask, d["cu_seqlens"]), (labels, mask.clone())


@BATCH_FN_REGISTRY.register("mini_rlhf_json_batch_pipe")
class MiniRLHFJsonBatchFunction(JsonBatchFunction):
    def __call__(self, data):
        inputs, (labels, loss_mask) = super().__call__(data)
        if get_grid().tp > 1:
            scores = broadcast_data(["scores"], {"scores": data["scores"].float()} if data is not None else None,
                                    torch.float32)["scores"]
        else:
            scores = data["scores"].float().to(labels.device)
        return inputs, (labels, loss_mask, scores)


@BATCH_FN_REGISTRY.register("token_batch_pipe")
class TokenBatchFunction(_PipeBase):
    """Inference: a flat tensor of prompt tokens → one micro-batch (labels = next tokens)."""

    def __init__(self, tokenizer, reset_position_ids=False, reset_attention_mask=False, eod_mask_loss=True,
                 prefix_indices=None, loss_on_targets_only=True, micro_batch_size=1):
        super().__init__(tokenizer)
        self.a = (reset_position_ids, reset_attention_mask, eod_mask_loss, prefix_indices, loss_on_targets_only)
        self.micro_batch_size = micro_batch_size

    def __call__(self, data):
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        tokens = data.view(self.micro_batch_size, -1).contiguous().to(dev)
        eos = self.tokenizer.eos_token_id
        labels = torch.cat([tokens[:, 1:], tokens.new_full((tokens.shape[0], 1), eos)], dim=-1)
        mask, loss_mask, pos, cu = get_ltor_masks_and_position_ids(tokens, eos, *self.a)
        inputs = (tokens, pos, mask) if cu is None else (tokens, pos, mask, cu)
        return inputs, (labels, loss_mask)


def build_batch_pipe_fn(cfg_batch_pipe, tokenizer):
    cfg = {"type": cfg_batch_pipe["type"], "kwargs": dict(cfg_batch_pipe.get("kwargs") or {})}
    cfg["kwargs"]["tokenizer"] = tokenizer
    return BATCH_FN_REGISTRY.build(cfg)


class _NoneIterator:
    """What non-loading TP ranks iterate: the batch function receives ``None`` and gets the data
    by broadcast."""

    def __iter__(self):
        return self

    def __next__(self):
        return None


def build_data_iterator(tokenizer, cfg_data, consumed_train_samples=0, data_type="train"):
    """Returns (iterator, dataset_size).  Only TP rank 0 builds the dataset/loader; the size is
    broadcast to the TP group."""
    g = get_grid()
    cfg = cfg_data[data_type]
    size = torch.zeros(1, dtype=torch.int64)
    it = None
    if g.tp_rank == 0:
        dataset = build_dataset(cfg["dataset"], tokenizer)
        bs_cfg = {"type": cfg["batch_sampler"]["type"], "kwargs": dict(cfg["batch_sampler"].get("kwargs") or {})}
        bs_cfg["kwargs"].update(total_samples=len(dataset), data_parallel_rank=g.dp_rank, data_parallel_size=g.dp)
        bs_cfg["kwargs"].setdefault("micro_batch_size", cfg["micro_batch_size"])
        if bs_cfg["type"] != "base":
            bs_cfg["kwargs"]["consumed_samples"] = consumed_train_samples
        sampler = build_batch_sampler(bs_cfg)
        if bs_cfg["type"] == "base" and hasattr(sampler, "set_consumed_samples"):
            sampler.set_consumed_samples(consumed_train_samples)
        collator = build_batch_collator(cfg["batch_collector"], tokenizer)
        loader = build_data_loader(cfg.get("data_loader", {"type": "base"}), dataset, sampler, collator)
        it = iter(loader)
        size[0] = len(dataset)
    if g.tp > 1:
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        size = size.to(dev)
        dist.broadcast(size, g.tp_src_rank(), group=g.tp_group)
    if it is None:
        it = _NoneIterator()
    return it, int(size.item())
