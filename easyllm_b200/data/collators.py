"""Batch collators (llm/data/nlp_dataloader.py:18-213).

``batch`` pads to the longest sample; ``batch_align`` pads to a multiple of ``alignment``
(sequence parallelism needs the length divisible by TP) and **shifts labels by one** when
``offset_label`` (the megatron runner's convention: the collator, not the model, aligns
targets); in ``pretrain`` mode it also carries per-sample ``cu_seqlens`` flattened with a
``sample_index · max_seq_length`` offset and per-document ``position_ids``.  ``reward_batch``
stacks (chosen, rejected) pairs, ``mini_rlhf_batch`` flattens answer groups and their scores.
The pad id is ``len(tokenizer) − 1`` everywhere.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import BATCH_COLLECTOR_REGISTRY


def _pad_stack(seqs, value, length):
    out = torch.full((len(seqs), length), value, dtype=torch.long)
    for i, s in enumerate(seqs):
        n = min(len(s), length)
        out[i, :n] = torch.as_tensor(s[:n], dtype=torch.long)
    return out


@BATCH_COLLECTOR_REGISTRY.register("batch")
class BatchCollector:
    def __init__(self, tokenizer, ignore_idx=-100, max_seq_length=2048, offset_label=False):
        self.tokenizer, self.ignore_idx, self.max_seq_length = tokenizer, ignore_idx, max_seq_length
        self.pad_token_id = len(tokenizer) - 1
        self.offset_label = offset_label

    def _pad_func(self, input_ids, labels):
        n = max(len(x) for x in input_ids)
        ids = _pad_stack(input_ids, self.pad_token_id, n)
        lab = _pad_stack(labels, self.ignore_idx, n)
        if self.offset_label:
            ids, lab = ids[:, :-1], lab[:, 1:]
        return ids[:, :self.max_seq_length].contiguous(), lab[:, :self.max_seq_length].contiguous()

    def __call__(self, instances):
        ids, lab = self._pad_func([i["input_ids"] for i in instances], [i["labels"] for i in instances])
        return dict(input_ids=ids, labels=lab, attention_mask=ids.ne(self.pad_token_id))


@BATCH_COLLECTOR_REGISTRY.register("batch_align")
class BatchAlignCollector(BatchCollector):
    def __init__(self, tokenizer, alignment=1, ignore_idx=-100, max_seq_length=2048, offset_label=True,
                 test_speed=False, pretrain=False):
        super().__init__(tokenizer, ignore_idx, max_seq_length, offset_label)
        self.alignment, self.test_speed, self.pretrain = alignment, test_speed, pretrain

    def _aligned(self, seqs, value, is_label=False):
        if self.test_speed:
            value = 100                       # speed tests train on every position
        longest = max(len(s) for s in seqs)
        width = min(self.max_seq_length, math.ceil(longest / float(self.alignment)) * self.alignment)
        out = torch.full((len(seqs), width), value, dtype=torch.long)
        for i, s in enumerate(seqs):
            s = torch.as_tensor(s, dtype=torch.long)
            if self.offset_label:
                s = s[1:] if is_label else s[:-1]
            n = min(len(s), width)
            out[i, :n] = s[:n]
        return out

    def _pad_func(self, input_ids, labels, cu_seqlens=None, position_ids=None):
        ids = self._aligned(input_ids, self.pad_token_id)
        lab = self._aligned(labels, self.ignore_idx, is_label=True)
        if not self.pretrain:
            return ids, lab
        pos = self._aligned(position_ids, 0)
        flat = []
        for b, cu in enumerate(cu_seqlens):
            cu = torch.clamp(torch.as_tensor(cu, dtype=torch.long), max=self.max_seq_length) + b * self.max_seq_length
            flat.append(cu if b == 0 else cu[1:])
        return ids, lab, torch.cat(flat), pos

    def __call__(self, instances):
        ids = [i["input_ids"] for i in instances]
        lab = [i["labels"] for i in instances]
        if self.pretrain:
            ids, lab, cu, pos = self._pad_func(ids, lab, [i["cu_seqlens"] for i in instances],
                                               [i["position_ids"] for i in instances])
            return dict(input_ids=ids, labels=lab, attention_mask=ids.ne(self.pad_token_id), cu_seqlens=cu,
                        position_ids=pos)
        ids, lab = self._pad_func(ids, lab)
        return dict(input_ids=ids, labels=lab, attention_mask=ids.ne(self.pad_token_id))


@BATCH_COLLECTOR_REGISTRY.register("reward_batch")
class RewardBatchCollector:
    def __init__(self, tokenizer, ignore_idx=-100, max_seq_length=2048):
        self.tokenizer, self.ignore_idx, self.max_seq_length = tokenizer, ignore_idx, max_seq_length
        self.pad_token_id = len(tokenizer) - 1

    def __call__(self, instances):
        chosen = [i["input_ids"][0] for i in instances]
        rejected = [i["input_ids"][1] for i in instances]
        width = min(self.max_seq_length, max(len(x) for x in chosen + rejected))
        ids = torch.cat((_pad_stack(chosen, self.pad_token_id, width), _pad_stack(rejected, self.pad_token_id, width)))
        lab = torch.cat((_pad_stack(chosen, self.ignore_idx, width), _pad_stack(rejected, self.ignore_idx, width)))
        return dict(input_ids=ids, labels=lab, attention_mask=ids.ne(self.pad_token_id))


@BATCH_COLLECTOR_REGISTRY.register("mini_rlhf_batch")
class MiniRLHFBatchCollector(BatchAlignCollector):
    def __init__(self, tokenizer, alignment=1, ignore_idx=-100, max_seq_length=2048, pad_type="right", **kw):
        super().__init__(tokenizer, alignment, ignore_idx, max_seq_length, **kw)

    def __call__(self, instances):
        ids = [x for i in instances for x in i["input_ids"]]
        lab = [x for i in instances for x in i["labels"]]
        ids, lab = self._pad_func(ids, lab)
        return dict(input_ids=ids, labels=lab, scores=torch.cat([i["scores"] for i in instances], dim=0),
                    attention_mask=ids.ne(self.pad_token_id))
