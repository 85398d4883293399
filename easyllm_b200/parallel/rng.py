"""Seeding and the model-parallel RNG tracker.

Parity: llm/utils/env/gene_env.py:78-91 (seed + 100·pp_rank, optional +3·dp_rank) and the
CUDA RNG tracker the reference borrows from DeepSpeed's activation checkpointing: a named
set of generator states so tensor-parallel-sharded weights are initialised from a
per-TP-rank stream (seed + 2718 + tp_rank) while replicated tensors use the default stream.
Works on CPU generators too, which is what the gloo tests run.
"""
from __future__ import annotations

import contextlib
import random

import numpy as np
import torch

from .grid import get_grid

_MP_RNG = "model-parallel-rng"


class RNGStatesTracker:
    def __init__(self):
        self.states = {}
        self.seeds = set()

    def reset(self):
        self.states.clear()
        self.seeds.clear()

    def get_states(self):
        return dict(self.states)

    def set_states(self, states):
        self.states = dict(states)

    @staticmethod
    def _get():
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    @staticmethod
    def _set(s):
        if torch.cuda.is_available():
            torch.cuda.set_rng_state(s)
        else:
            torch.set_rng_state(s)

    def add(self, name, seed):
        if seed in self.seeds:
            raise ValueError(f"seed {seed} already present")
        if name in self.states:
            raise ValueError(f"rng state {name} already present")
        self.seeds.add(seed)
        keep = self._get()
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states[name] = self._get()
        self._set(keep)

    @contextlib.contextmanager
    def fork(self, name=_MP_RNG):
        if name not in self.states:
            yield
            return
        keep = self._get()
        self._set(self.states[name])
        try:
            yield
        finally:
            self.states[name] = self._get()
            self._set(keep)


_TRACKER = RNGStatesTracker()


def get_rng_tracker():
    return _TRACKER


get_cuda_rng_tracker = get_rng_tracker


def model_parallel_manual_seed(seed):
    g = get_grid()
    _TRACKER.reset()
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _TRACKER.add(_MP_RNG, seed + 2718 + g.tp_rank)


def set_random_seed(seed, dp_random_init=False):
    if seed is None or seed <= 0:
        raise ValueError(f"seed must be a positive integer, got {seed}")
    g = get_grid()
    seed = seed + 100 * g.pp_rank
    if dp_random_init:
        seed = seed + 3 * g.dp_rank
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    model_parallel_manual_seed(seed)
    return seed
