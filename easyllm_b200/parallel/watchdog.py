"""Host-side failure detection: heartbeats over a TCP store, NaN policy, bounded-wait status.

The reference relies on ``NCCL_ASYNC_ERROR_HANDLING=1`` and scheduler requeue
(scripts/mg_infer.sh:51-52, hook_helper.py:196-222); nothing detects a dead or hung rank.
Here every rank runs a daemon thread that bumps ``hb/<rank>`` in a ``TCPStore`` every
``interval`` seconds and checks its peers' counters; a peer whose counter has not moved for
``timeout`` seconds is reported through ``on_failure`` (default: log, set ``failed_ranks``, and
make the next ``check()`` raise ``RankFailure`` on the training thread — between steps, with
no collective in flight).  Device-side waits are bounded inside the kernels themselves and
surface through ``ops.cuda.check_err_flag``; ``check()`` reads that word too.
Failures are *made* on the host in tests (a rank that exits or stops beating); no GPU is ever
faulted to exercise this path.
"""
from __future__ import annotations

import datetime
import os
import threading
import time

import torch.distributed as dist


class RankFailure(RuntimeError):
    pass


class Watchdog:
    def __init__(self, rank, world, store=None, host="127.0.0.1", port=None, interval=1.0, timeout=10.0,
                 on_failure=None, check_device_flag=False):
        self.rank, self.world, self.interval, self.timeout = rank, world, interval, timeout
        if store is None:
            port = port or int(os.environ.get("MASTER_PORT", "29500")) + 17
            store = dist.TCPStore(host, port, world, rank == 0, timeout=datetime.timedelta(seconds=60),
                                  wait_for_workers=False)
        self.store = store
        self.on_failure = on_failure
        self.failed_ranks = set()
        self.left_ranks = set()
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._thread = None
        self._beat = 0
        self._last_seen = {}
        self.check_device_flag = check_device_flag

    def start(self):
        self.store.set(f"hb/{self.rank}", "0")
        now = time.time()
        self._last_seen = {r: (None, now) for r in range(self.world)}
        self._thread = threading.Thread(target=self._run, name="easyllm-watchdog", daemon=True)
        self._thread.start()
        return self

    def _run(self):
        while not self._stop.wait(self.interval):
            if not self._paused.is_set():
                self._beat += 1
                try:
                    self.store.set(f"hb/{self.rank}", str(self._beat))
                except Exception:
                    return
            now = time.time()
            for r in range(self.world):
                if r == self.rank or r in self.failed_ranks or r in self.left_ranks:
                    continue
                try:
                    if self.store.check([f"left/{r}"]):
                        self.left_ranks.add(r)
                        continue
                    val = self.store.get(f"hb/{r}").decode() if self.store.check([f"hb/{r}"]) else None
                except Exception:
                    val = None
                prev, since = self._last_seen.get(r, (None, now))
                if val is not None and val != prev:
                    self._last_seen[r] = (val, now)
                elif now - since > self.timeout:
                    self.failed_ranks.add(r)
                    if self.on_failure is not None:
                        self.on_failure(r)

    def pause_heartbeat(self, flag=True):
        """Test hook: stop beating without leaving (simulates a hung rank)."""
        (self._paused.set if flag else self._paused.clear)()

    def check(self):
        """Call between steps on the training thread; raises if a peer failed or a kernel gave up a wait."""
        if self.failed_ranks:
            raise RankFailure(f"rank(s) {sorted(self.failed_ranks)} stopped sending heartbeats "
                              f"(> {self.timeout:.0f} s); stopping before the next collective")
        if self.check_device_flag:
            from ..ops import cuda
            cuda.check_err_flag()

    def leave(self):
        """Graceful departure between steps: peers stop monitoring this rank."""
        try:
            self.store.set(f"left/{self.rank}", "1")
        except Exception:
            pass
        self.stop()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
