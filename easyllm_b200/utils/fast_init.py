"""Fast model construction (llm/utils/general/fast_init.py:10-54): while the context is active,
``nn.Linear`` / ``nn.Embedding`` / ``nn.LayerNorm`` allocate on the ``meta`` device and skip their
random initialisation; on exit the module tree is materialised with ``to_empty(device)`` by the
caller.  Used when weights are about to be overwritten by a checkpoint."""
from __future__ import annotations

import contextlib

import torch.nn as nn


@contextlib.contextmanager
def fast_init(device="meta", skip_init=True):
    saved = {}
    classes = (nn.Linear, nn.Embedding, nn.LayerNorm)

    def wrap(cls):
        orig = cls.__init__

        def init(self, *a, **k):
            k.setdefault("device", device)
            if skip_init and hasattr(self, "reset_parameters"):
                rp = cls.reset_parameters
                cls.reset_parameters = lambda self: None
                try:
                    orig(self, *a, **k)
                finally:
                    cls.reset_parameters = rp
            else:
                orig(self, *a, **k)
        saved[cls] = orig
        cls.__init__ = init
    for c in classes:
        wrap(c)
    try:
        yield
    finally:
        for c, o in saved.items():
            c.__init__ = o


def materialize(model, device):
    return model.to_empty(device=device) if any(p.is_meta for p in model.parameters()) else model.to(device)
