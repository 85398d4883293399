"""Name → factory registries; components are selected in YAML by ``{type, kwargs}``.

Parity: llm/utils/general/registry.py:19-130 and registry_factory.py:4-28 (the 14 global
registries).  ``REGTRACE=ON`` records the registering file:line for ``query_details``.
Unknown types raise on rank 0 and exit(1) elsewhere so a typo does not print N tracebacks.
"""
from __future__ import annotations

import inspect
import os
import sys
from collections import OrderedDict

_TRACE = os.environ.get("REGTRACE", "OFF").upper() == "ON"


def _rank():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:
        pass
    return 0


class Registry(dict):
    def __init__(self, name="registry", *a, **kw):
        super().__init__(*a, **kw)
        self.name = name
        self._trace = {}

    def register(self, module_name=None, module=None):
        where = None
        if _TRACE:
            fr = inspect.stack()[1]
            where = (fr.filename, fr.lineno)

        def _add(name, obj):
            if name in self:
                raise KeyError(f"{self.name}: duplicate registration of {name!r}")
            self[name] = obj
            if where:
                self._trace[name] = where

        if module is not None:
            if module_name is None:
                raise ValueError("register(name, obj) needs a name")
            _add(module_name, module)
            return module

        def deco(fn):
            _add(module_name or fn.__name__, fn)
            return fn

        return deco

    def get(self, name, default=None):
        if name not in self:
            if default is not None:
                return default
            self._unknown(name)
        return self[name]

    def _unknown(self, name):
        if _rank() == 0:
            raise KeyError(f"{self.name}: {name!r} is not supported; available: {sorted(self.keys())}")
        sys.exit(1)

    def build(self, cfg):
        kind = cfg["type"]
        kwargs = cfg.get("kwargs") or {}
        if kind not in self:
            self._unknown(kind)
        fn = self[kind]
        try:
            return fn(**kwargs)
        except TypeError as e:
            try:
                spec = inspect.signature(fn)
            except (TypeError, ValueError):
                spec = "?"
            raise TypeError(f"{self.name}.build({kind!r}): {e}\n  expected {spec}\n  given {sorted(kwargs)}") from e

    def query(self):
        return self.keys()

    def query_details(self, aliases=None):
        if not _TRACE:
            raise RuntimeError("export REGTRACE=ON before importing to record registration sites")
        return OrderedDict((a, self._trace[a]) for a in (aliases or self.keys()))


TOKENIZER_REGISTRY = Registry("TOKENIZER")
BATCH_CALCULATOR_REGISTRY = Registry("BATCH_CALCULATOR")
DATASET_REGISTRY = Registry("DATASET")
PARSER_REGISTRY = Registry("PARSER")
AUGMENTATION_REGISTRY = Registry("AUGMENTATION")
BATCH_COLLECTOR_REGISTRY = Registry("BATCH_COLLECTOR")
SAMPLER_REGISTRY = Registry("SAMPLER")
BATCH_SAMPLER_REGISTRY = Registry("BATCH_SAMPLER")
DATALOADER_REGISTRY = Registry("DATALOADER")
BATCH_FN_REGISTRY = Registry("BATCH_FN")
LR_REGISTRY = Registry("LR")
MODULE_ZOO_REGISTRY = Registry("MODULE_ZOO")
HOOK_REGISTRY = Registry("HOOK")
LOSS_REGISTRY = Registry("LOSS")
