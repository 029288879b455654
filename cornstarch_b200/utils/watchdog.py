"""Failure detection on the host: a per-step watchdog and a store-based heartbeat between ranks.

The reference has no failure detector (its only remnants of elastic training are the tensor placeholders and
``HeterogeneousParallelPlugin.configure(forced=True)``, cornstarch/shardformer/shard/shardformer.py:47-111 and
cornstarch/plugin/heterogeneous_parallel_plugin/heterogeneous_parallel_plugin.py:186-277).  Two host-side pieces
complete the picture here; neither touches GPU settings or resets anything:

* :class:`StepWatchdog` - a thread that polls a CUDA event recorded at the end of each step (``event.query()``,
  i.e. ``cudaEventQuery``) and the library's device status word.  A step that does not finish within the deadline,
  or a kernel that gave up a bounded wait (the status word names which), is reported through a callback; the
  training loop decides what to do (save and exit, re-plan).  On CPU the "event" is a plain flag.
* :class:`Heartbeat` - every rank bumps ``hb/<rank>`` in a ``torch.distributed`` store from a thread; a rank whose
  counter stops for longer than the timeout is reported as failed by everyone else *before their next launch*,
  so no collective is entered with a dead peer.  ``survivors()`` is the input of a re-plan
  (``HeterogeneousParallelPlugin.set_pipelines`` + ``configure(forced=True)``).
"""

from __future__ import annotations

import threading
import time
from typing import Callable

import torch


class StepWatchdog:
    def __init__(self, deadline_s: float, on_timeout: Callable[[dict], None] | None = None, poll_s: float = 0.05,
                 status_reader: Callable[[], int] | None = None):
        self.deadline_s, self.poll_s = deadline_s, poll_s
        self.on_timeout = on_timeout or (lambda info: None)
        self.status_reader = status_reader
        self._lock = threading.Lock()
        self._armed_at: float | None = None
        self._event = None
        self._step = -1
        self._stop = threading.Event()
        self.reports: list[dict] = []
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def arm(self, step: int, done_flag=None):
        """Call after the step's work has been enqueued.  ``done_flag``: a ``torch.cuda.Event`` (recorded here on the
        current stream when ``None`` and CUDA is in use) or any object with ``query() -> bool``."""
        if done_flag is None and torch.cuda.is_available():
            done_flag = torch.cuda.Event()
            done_flag.record()
        with self._lock:
            self._event, self._step, self._armed_at = done_flag, step, time.monotonic()

    def disarm(self):
        with self._lock:
            self._armed_at = None

    def _run(self):
        while not self._stop.wait(self.poll_s):
            with self._lock:
                armed, ev, step = self._armed_at, self._event, self._step
            if armed is None:
                continue
            done = ev.query() if ev is not None else False
            status = self.status_reader() if self.status_reader else 0
            if status:
                self._report({"step": step, "reason": "device_status", "status": int(status)})
            elif done:
                self.disarm()
            elif time.monotonic() - armed > self.deadline_s:
                self._report({"step": step, "reason": "deadline", "elapsed_s": time.monotonic() - armed})

    def _report(self, info: dict):
        self.disarm()
        self.reports.append(info)
        self.on_timeout(info)

    def close(self):
        self._stop.set()
        self._thread.join(timeout=2)


class Heartbeat:
    """Liveness of the ranks of a job through a key-value store (``dist.TCPStore`` / ``FileStore`` / ``HashStore``)."""

    def __init__(self, store, rank: int, world: int, interval_s: float = 0.2, timeout_s: float = 2.0):
        self.store, self.rank, self.world = store, rank, world
        self.interval_s, self.timeout_s = interval_s, timeout_s
        self._stop = threading.Event()
        self._beats = 0
        self._seen: dict[int, tuple[int, float]] = {}
        self.store.set(f"hb/{rank}", "0")
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.wait(self.interval_s):
            self._beats += 1
            try:
                self.store.set(f"hb/{self.rank}", str(self._beats))
            except Exception:  # noqa: BLE001  (store owner gone: nothing more to publish)
                return

    def failed(self) -> list[int]:
        """Ranks whose counter has not moved for ``timeout_s`` (never-seen ranks count from the first look)."""
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = int(self.store.get(f"hb/{r}").decode()) if self.store.check([f"hb/{r}"]) else -1
            except Exception:  # noqa: BLE001
                val = -1
            last = self._seen.get(r)
            if last is None or val != last[0]:
                self._seen[r] = (val, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead

    def survivors(self) -> list[int]:
        dead = set(self.failed())
        return [r for r in range(self.world) if r not in dead]

    def check(self):
        """Raise before the next launch if a peer is gone."""
        dead = self.failed()
        if dead:
            raise PeerFailure(dead)

    def stop(self):
        self._stop.set()
        self._thread.join(timeout=2)


class PeerFailure(RuntimeError):
    def __init__(self, ranks: list[int]):
        super().__init__(f"ranks {ranks} stopped sending heartbeats")
        self.ranks = ranks
