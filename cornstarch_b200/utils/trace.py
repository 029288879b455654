"""NVTX ranges around the schedule phases and the optimizer, for timelines taken with an external profiler.

The reference has no NVTX ranges or profiler hooks (only the ``TimerContextManager`` / ``DcgmContextManager``
benchmarking aids, cornstarch/testing/timer.py:11-128, cornstarch/testing/dcgm.py:12-107).  Ranges are off by
default (a range push / pop costs a little host time on every micro-batch); ``CORNSTARCH_B200_NVTX=1`` or
``enable(True)`` turns them on.  Without CUDA the context manager does nothing, and ``recorded`` keeps the names so
that the placement of the ranges can be tested on CPU.

The same ranges can be timed on the device: ``timeline(True)`` makes every range record a pair of CUDA events on the
current stream, and ``timeline_totals()`` returns ``{range name: (count, total ms)}``.  A range around a wait for a
received tensor then measures how long the compute stream stood still for it (``bench.py`` writes the per-rank totals of a
pipeline step to the file named by ``CORNSTARCH_B200_TIMELINE``).
"""

from __future__ import annotations

import contextlib
import os

import torch

_enabled = os.environ.get("CORNSTARCH_B200_NVTX", "0") == "1"
recorded: list[str] | None = None  # set to a list to collect range names (tests)


_timeline = False
_events: dict[str, list] = {}


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on


def timeline(on: bool = True) -> None:
    """Record CUDA events around every range from now on (or stop doing so); forgets what was recorded before."""
    global _timeline
    _timeline = on and torch.cuda.is_available()
    _events.clear()


def timeline_totals() -> dict[str, tuple[int, float]]:
    """``{range name: (count, total device milliseconds)}`` of the ranges recorded since ``timeline(True)``; synchronises."""
    if not _events:
        return {}
    torch.cuda.synchronize()
    out = {name: (len(pairs), sum(a.elapsed_time(b) for a, b in pairs)) for name, pairs in _events.items()}
    _events.clear()
    return out


@contextlib.contextmanager
def nvtx_range(name: str):
    if recorded is not None:
        recorded.append(name)
    if _timeline:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        try:
            yield
        finally:
            b.record()
            _events.setdefault(name, []).append((a, b))
        return
    if not (_enabled and torch.cuda.is_available()):
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
