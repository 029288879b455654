"""NVTX ranges around the schedule phases and the optimizer, for timelines taken with an external profiler.

The reference has no NVTX ranges or profiler hooks (only the ``TimerContextManager`` / ``DcgmContextManager``
benchmarking aids, cornstarch/testing/timer.py:11-128, cornstarch/testing/dcgm.py:12-107).  Ranges are off by
default (a range push / pop costs a little host time on every micro-batch); ``CORNSTARCH_B200_NVTX=1`` or
``enable(True)`` turns them on.  Without CUDA the context manager does nothing, and ``recorded`` keeps the names so
that the placement of the ranges can be tested on CPU.
"""

from __future__ import annotations

import contextlib
import os

import torch

_enabled = os.environ.get("CORNSTARCH_B200_NVTX", "0") == "1"
recorded: list[str] | None = None  # set to a list to collect range names (tests)


def enable(on: bool = True) -> None:
    global _enabled
    _enabled = on


@contextlib.contextmanager
def nvtx_range(name: str):
    if recorded is not None:
        recorded.append(name)
    if not (_enabled and torch.cuda.is_available()):
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()
