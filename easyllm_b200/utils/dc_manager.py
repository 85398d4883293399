"""Dynamic Checkpoint for module-tree (HuggingFace-style) models.

Parity: llm/utils/general/dc_manager.py:6-110 and the ``dynamic_checkpoint`` hook
(llm/utils/general/hf_hook_helper.py:11-142).  Candidate modules are found breadth-first at
the depth of the ``level_keys`` containers (default ``"layers"``; embeddings and in-place
modules excluded).  Each candidate's ``forward`` is wrapped so it runs under
``torch.utils.checkpoint`` iff its name is in the set chosen for the current input size; per
iteration the first ``size_map[bucket(seq_len × batch)]`` candidates are recomputed (keys
are sequence lengths, scaled by the batch size; larger inputs than any key use the last key).
The Megatron form of the policy lives in ``models.llama.LlamaModelPipe.recompute_plan``.
"""
from __future__ import annotations

import functools

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .log import default_logger as logger


def bfs_candidates(model, level_keys=("layers",), exclude=(nn.Embedding,)):
    """Names of the children of every module whose attribute name is in ``level_keys``."""
    out, frontier = [], [("", model)]
    while frontier:
        nxt = []
        for prefix, mod in frontier:
            for name, child in mod.named_children():
                full = f"{prefix}.{name}" if prefix else name
                if name in level_keys:
                    for cn, cm in child.named_children():
                        if not isinstance(cm, tuple(exclude)) and not getattr(cm, "inplace", False):
                            out.append(f"{full}.{cn}")
                else:
                    nxt.append((full, child))
        if out:
            break
        frontier = nxt
    return out


class DynamicCheckpointManager:
    def __init__(self, model, size_map, level_keys=("layers",), debug=False):
        self.model = model
        self.size_map = {int(k): int(v) for k, v in size_map.items()}
        self.keys = sorted(self.size_map)
        self.candidates = bfs_candidates(model, tuple(level_keys))
        self.cur_checkpoint_modules = set()
        self.cache = {}
        self.debug = debug
        self._wrap()

    def _wrap(self):
        mods = dict(self.model.named_modules())
        for name in self.candidates:
            m = mods[name]
            if getattr(m, "_dc_wrapped", False):
                continue
            orig = m.forward

            @functools.wraps(orig)
            def fwd(*a, __name=name, __orig=orig, **k):
                if __name in self.cur_checkpoint_modules and torch.is_grad_enabled():
                    return checkpoint(__orig, *a, use_reentrant=False, **k)
                return __orig(*a, **k)
            m.forward = fwd
            m._dc_wrapped = True

    def num_to_checkpoint(self, seq_len, batch=1):
        size = seq_len * batch
        for k in self.keys:
            if size <= k * batch:
                return self.size_map[k]
        return self.size_map[self.keys[-1]]

    def before_forward(self, input_ids):
        batch, seq = input_ids.shape[0], input_ids.shape[-1]
        key = (batch, seq)
        if key not in self.cache:
            n = self.num_to_checkpoint(seq, batch)
            n = len(self.candidates) if n < 0 else min(n, len(self.candidates))
            self.cache[key] = set(self.candidates[:n])
            if self.debug:
                logger.info(f"dynamic checkpoint: input {key} -> recompute {n}/{len(self.candidates)} modules")
        self.cur_checkpoint_modules = self.cache[key]
        return len(self.cur_checkpoint_modules)
