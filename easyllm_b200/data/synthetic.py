"""Synthetic token data of a named shape (benchmarks and parity tests; no dataset files).

Samples are uniform random token ids from a fixed seed, labels are the ids shifted by one
(the collator convention of the megatron runner: ``offset_label``).  ``packed_varlen=True``
produces variable-length documents drawn uniformly from ``[min_len, max_len]`` and packed up
to ``seq_length`` tokens with ``cu_seqlens`` and per-document position ids.
"""
from __future__ import annotations

import torch

from ..parallel.grid import get_grid


class SyntheticTokenDataset(torch.utils.data.Dataset):
    def __init__(self, vocab_size, seq_length, num_samples=1 << 20, seed=0):
        self.vocab_size, self.seq_length, self.num_samples, self.seed = vocab_size, seq_length, num_samples, seed

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.seed * 1000003 + idx)
        ids = torch.randint(0, self.vocab_size, (self.seq_length + 1,), generator=g, dtype=torch.int64)
        return {"input_ids": ids[:-1], "labels": ids[1:].clone()}


def synthetic_batches(vocab_size, seq_length, micro_batch_size, seed=0, dp_rank=None, dp_size=None,
                      packed_varlen=False, min_len=256, max_len=None, pin=False, start=0):
    """Infinite iterator of ``((tokens, position_ids, None[, cu_seqlens]), (labels, loss_mask))``
    CPU tensors for this data-parallel rank (sample i of the global stream goes to rank
    ``i mod dp`` within each group of ``dp`` consecutive samples)."""
    g = get_grid()
    dp_rank = g.dp_rank if dp_rank is None else dp_rank
    dp_size = g.dp if dp_size is None else dp_size
    ds = SyntheticTokenDataset(vocab_size, seq_length, seed=seed)
    step = start
    max_len = max_len or seq_length

    def maybe_pin(t):
        return t.pin_memory() if pin and torch.cuda.is_available() else t

    while True:
        rows = [ds[(step * dp_size + dp_rank) * micro_batch_size + j] for j in range(micro_batch_size)]
        step += 1
        tok = torch.stack([r["input_ids"] for r in rows])
        lab = torch.stack([r["labels"] for r in rows])
        mask = torch.ones_like(lab)
        if not packed_varlen:
            pos = torch.arange(seq_length, dtype=torch.int64).unsqueeze(0).repeat(micro_batch_size, 1)
            yield (maybe_pin(tok), maybe_pin(pos), None), (maybe_pin(lab), maybe_pin(mask))
            continue
        gen = torch.Generator().manual_seed(seed * 7919 + step)
        cu, pos = [0], torch.empty(micro_batch_size, seq_length, dtype=torch.int64)
        for b in range(micro_batch_size):
            at = 0
            while at < seq_length:
                n = int(torch.randint(min_len, max_len + 1, (1,), generator=gen))
                n = min(n, seq_length - at)
                pos[b, at:at + n] = torch.arange(n)
                mask[b, at + n - 1] = 0          # do not predict across a document boundary
                at += n
                cu.append(b * seq_length + at)
        cu_t = torch.tensor(cu, dtype=torch.int32)
        yield (maybe_pin(tok), maybe_pin(pos), None, maybe_pin(cu_t)), (maybe_pin(lab), maybe_pin(mask))
