"""Timers and memory reports.

Parity: llm/utils/general/utils.py:9-107 (named wall-clock timers that synchronise the
device around start/stop; ``report_memory``).  Added: ``DeviceTimer`` which measures with
CUDA events on the launching stream, the form used for every benchmark number.
"""
from __future__ import annotations

import time

import torch


def _sync():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


class _Timer:
    def __init__(self, name):
        self.name = name
        self.total = 0.0
        self.running = False
        self.t0 = 0.0

    def start(self):
        if self.running:
            raise RuntimeError(f"timer {self.name} already started")
        _sync()
        self.t0 = time.time()
        self.running = True

    def stop(self):
        if not self.running:
            raise RuntimeError(f"timer {self.name} is not started")
        _sync()
        self.total += time.time() - self.t0
        self.running = False

    def reset(self):
        self.total = 0.0
        self.running = False

    def elapsed(self, reset=True):
        was = self.running
        if was:
            self.stop()
        out = self.total
        if reset:
            self.reset()
        if was:
            self.start()
        return out


class Timers:
    def __init__(self):
        self.timers = {}

    def __call__(self, name):
        if name not in self.timers:
            self.timers[name] = _Timer(name)
        return self.timers[name]

    def write(self, names, writer, iteration, normalizer=1.0, reset=False):
        for n in names:
            writer.add_scalar(f"time/{n}-time", self.timers[n].elapsed(reset=reset) / normalizer, iteration)

    def log(self, names, normalizer=1.0, reset=True):
        parts = [f"{n}: {self.timers[n].elapsed(reset=reset) * 1000.0 / normalizer:.2f}" for n in names]
        if parts:
            print("time (ms) | " + " | ".join(parts), flush=True)


class DeviceTimer:
    """CUDA-event timer; ``ms()`` synchronises and returns the elapsed milliseconds."""

    def __init__(self):
        self.a = torch.cuda.Event(enable_timing=True)
        self.b = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.a.record()
        return self

    def __exit__(self, *exc):
        self.b.record()

    def ms(self):
        self.b.synchronize()
        return self.a.elapsed_time(self.b)


def report_memory(name, printer=print):
    if not torch.cuda.is_available():
        return ""
    mb = 1024.0 * 1024.0
    s = (f"{name} memory (MB) | allocated: {torch.cuda.memory_allocated() / mb:.1f}"
         f" | max allocated: {torch.cuda.max_memory_allocated() / mb:.1f}"
         f" | reserved: {torch.cuda.memory_reserved() / mb:.1f}"
         f" | max reserved: {torch.cuda.max_memory_reserved() / mb:.1f}")
    printer(s)
    return s
