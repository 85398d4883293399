"""Rank-aware logging.

Parity: llm/utils/general/log_helper.py:35-89 — a process-wide logger named ``global``
that prints on stdout with ``<time>-rk<rank>-<file>#<line>:<message>`` and is silent on
every rank but 0 unless ``set_all_ranks(True)``.
"""
from __future__ import annotations

import logging
import os
import sys

_COLORS = {"WARNING": 33, "INFO": 0, "DEBUG": 34, "CRITICAL": 33, "ERROR": 31}
_all_ranks = False
_warned = set()


def _rank():
    try:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:
        pass
    return int(os.environ.get("RANK", 0))


def is_master():
    return _rank() == 0


def set_all_ranks(flag: bool):
    global _all_ranks
    _all_ranks = bool(flag)


class _Fmt(logging.Formatter):
    def __init__(self, color):
        super().__init__("%(asctime)s-rk%(rank)s-%(filename)s#%(lineno)d:%(message)s")
        self.color = color

    def format(self, record):
        record.rank = _rank()
        out = super().format(record)
        c = _COLORS.get(record.levelname, 0)
        if self.color and c:
            out = f"\033[1;{c}m{out}\033[0m"
        return out


def init_log(name="global", level=logging.INFO):
    logger = logging.getLogger(name)
    if getattr(logger, "_easyllm_ready", False):
        return logger
    logger.setLevel(level)
    h = logging.StreamHandler(stream=sys.stdout)
    h.setLevel(level)
    h.setFormatter(_Fmt(color=sys.stdout.isatty()))
    logger.addFilter(lambda rec: _all_ranks or is_master())
    logger.addHandler(h)
    logger.propagate = False
    logger._easyllm_ready = True

    def warning_once(msg, *a, **k):
        if msg not in _warned:
            _warned.add(msg)
            logger.warning(msg, *a, **k)

    logger.warning_once = warning_once
    return logger


default_logger = init_log()
