"""``TimerContextManager``: time any function, named by dotted path, with CUDA events.

Inside the context every call of a listed function (e.g. ``"torch.nn.functional.linear"`` or
``"cornstarch_b200.ops.attention.attention"``) is wrapped so that a ``torch.cuda.Event`` pair brackets
it on the current stream; the original function is restored on exit and ``get_elapsed_times()``
synchronises once and returns ``{path: [milliseconds, ...]}``.  On a machine without CUDA it falls back to
``time.perf_counter``.  Same contract as the reference aid (cornstarch/testing/timer.py:11-128).
"""

from __future__ import annotations

import importlib
import time
from typing import Callable

import torch


def _resolve(path: str):
    parts = path.split(".")
    for cut in range(len(parts) - 1, 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:cut]))
        except ImportError:
            continue
        owner = obj
        for name in parts[cut:-1]:
            owner = getattr(owner, name)
        return owner, parts[-1]
    raise ImportError(f"cannot resolve {path}")


class TimerContextManager:
    def __init__(self, *function_paths: str):
        self.paths = list(function_paths)
        self._originals: dict[str, tuple[object, str, Callable]] = {}
        self._events: dict[str, list] = {p: [] for p in self.paths}
        self._cuda = torch.cuda.is_available()

    def _wrap(self, path: str, fn: Callable) -> Callable:
        def timed(*a, **k):
            if self._cuda:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = fn(*a, **k)
                e.record()
                self._events[path].append((s, e))
            else:
                t0 = time.perf_counter()
                out = fn(*a, **k)
                self._events[path].append((time.perf_counter() - t0) * 1e3)
            return out

        timed.__wrapped__ = fn
        return timed

    def __enter__(self):
        for p in self.paths:
            owner, name = _resolve(p)
            fn = getattr(owner, name)
            self._originals[p] = (owner, name, fn)
            setattr(owner, name, self._wrap(p, fn))
        return self

    def __exit__(self, *exc):
        for owner, name, fn in self._originals.values():
            setattr(owner, name, fn)
        self._originals.clear()
        return False

    def get_elapsed_times(self) -> dict[str, list[float]]:
        if self._cuda:
            torch.cuda.synchronize()
            return {p: [s.elapsed_time(e) for s, e in evs] for p, evs in self._events.items()}
        return {p: list(v) for p, v in self._events.items()}
