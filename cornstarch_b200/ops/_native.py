"""ctypes binding of ``libcornstarch_b200.so`` (the hand-written sm_100a kernels).

The library has a plain C ABI: raw device pointers, sizes and a CUDA stream handle.  This module
loads it once, declares the prototypes, and offers small helpers to pass torch tensors.  On a machine
with a GPU the library is mandatory: :func:`lib` raises if it cannot be loaded, so GPU runs can never
fall back silently to eager PyTorch.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

# Library baseline: route every op to PyTorch / cuBLAS / cuDNN instead of this package's kernels (what the reference's
# call sites use); selected with CORNSTARCH_B200_LIBRARY_OPS=1 (bench.py --impl baseline) for same-box comparisons.
LIBRARY_MODE = os.environ.get("CORNSTARCH_B200_LIBRARY_OPS", "0") == "1"
_LIB = None
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libcornstarch_b200.so"

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_long, C.c_float

_PROTOS = {
    "csb_gemm_bf16": [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "csb_gemm_grouped_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "csb_norm_bwd_parts": [i32],
    "csb_norm_fwd": [i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, f32, f32, vp],
    "csb_norm_bwd": [i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, vp],
    "csb_colsum_parts": [i32],
    "csb_colsum": [vp, vp, vp, i32, i32, i32, i32, vp],
    "csb_rope": [vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, f32, i32, vp],
    "csb_glu_fwd": [vp, vp, i64, i32, i32, vp],
    "csb_glu_bwd": [vp, vp, vp, i64, i32, i32, vp],
    "csb_act_fwd": [vp, vp, i64, i32, vp],
    "csb_act_bwd": [vp, vp, vp, i64, i32, vp],
    "csb_add": [vp, vp, vp, i64, vp],
    "csb_adamw": [vp, vp, vp, vp, vp, i32, i64, f32, f32, f32, f32, f32, f32, f32, vp, vp, i32, vp],
    "csb_adamw_split": [vp, vp, vp, vp, vp, i32, i64, f32, f32, f32, f32, f32, f32, f32, vp, vp, i32, vp],
    "csb_sumsq": [vp, i32, i64, vp, vp, i32, vp],
    "csb_clip_scale": [vp, f32, f32, vp, vp, vp, vp, vp],
    "csb_mma_issue_probe": [i32, i32, i32, i32, vp, vp],
    "csb_ce_stats": [vp, i64, vp, i32, i32, vp, vp, vp, i64, vp],
    "csb_ce_grad": [vp, i64, vp, i32, i32, vp, vp, vp, vp, vp, i64, i64, vp],
    "csb_gather_merge": [vp, vp, vp, vp, i64, i32, i64, i64, vp],
    "csb_scatter_merge_bwd": [vp, vp, vp, i32, vp, i64, i32, i64, i64, vp],
}


def lib_path() -> Path:
    return Path(os.environ.get("CORNSTARCH_B200_LIB", str(_LIB_PATH)))


def available() -> bool:
    """True when the native library exists on disk and a CUDA device is present."""
    return torch.cuda.is_available() and lib_path().exists()


def lib():
    """Load (once) and return the native library; raises when it is missing."""
    global _LIB
    if _LIB is not None:
        return _LIB
    p = lib_path()
    if not p.exists():
        raise RuntimeError(
            f"native library {p} not found: run `python -m cornstarch_b200.csrc.build` "
            "(CUDA tensors never fall back to eager PyTorch)"
        )
    raw = C.CDLL(str(p))
    for name, args in _PROTOS.items():
        if hasattr(raw, name):
            fn = getattr(raw, name)
            fn.argtypes = args
            fn.restype = C.c_int
    _LIB = _CountingLib(raw)
    return _LIB


class _CountingLib:
    """Forwards attribute access to the CDLL and counts calls of kernel-launching entry points."""

    _NO_LAUNCH = {"csb_norm_bwd_parts", "csb_colsum_parts"}

    def __init__(self, raw):
        self._raw = raw
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            target = getattr(self._raw, name)
            if name in self._NO_LAUNCH:
                fn = target
            else:
                if KERNEL_TIMES:
                    def fn(*a, _t=target, _n=name):
                        global launch_count
                        launch_count += 1
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        r = _t(*a)
                        e1.record()
                        _TIMES.setdefault(_n, []).append((e0, e1))
                        return r
                else:
                    def fn(*a, _t=target):
                        global launch_count
                        launch_count += 1
                        return _t(*a)
            self._cache[name] = fn
        return fn


launch_count = 0
# CORNSTARCH_B200_KERNEL_TIMES=1: bracket every native call with a CUDA event pair on the launching stream and sum the
# device time per entry point (kernel_times()); a few microseconds of host time per call, for in-situ breakdowns.
KERNEL_TIMES = os.environ.get("CORNSTARCH_B200_KERNEL_TIMES", "0") == "1"
_TIMES: dict = {}


def kernel_times(reset: bool = True) -> dict:
    """``{entry point: (calls, total ms)}`` since the last reset (synchronises the device)."""
    torch.cuda.synchronize()
    out = {k: (len(v), sum(a.elapsed_time(b) for a, b in v)) for k, v in _TIMES.items()}
    if reset:
        _TIMES.clear()
    return out


def declare(name: str, argtypes: list) -> None:
    """Register the prototype of one more exported function (used by optional modules)."""
    _PROTOS[name] = argtypes
    if _LIB is not None and hasattr(_LIB._raw, name):
        fn = getattr(_LIB._raw, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int


def bounds_status() -> int:
    """Bounds-checked build of the library (``python -m cornstarch_b200.csrc.build --bounds-check``, loaded through
    ``CORNSTARCH_B200_LIB``): the first index violation a kernel recorded since the last call (0 = none), cleared by the
    call.  Always 0 with the release build.  Synchronises the device."""
    raw = lib()._raw
    raw.csb_bounds_status.restype = C.c_int
    return int(raw.csb_bounds_status())


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"cornstarch_b200 native call {what} failed with code {code}")


_STATUS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device int32 status word that kernels with bounded waits write on a time-out."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    t = _STATUS.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _STATUS[idx] = t
    return t


def status_in_use(device: torch.device | None = None) -> bool:
    """True once a kernel with bounded waits has been given this device's status word."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    return idx in _STATUS


_STATUS_NAMES = {1: "TMA stage never arrived", 2: "shared-memory slot never came back", 3: "accumulator never became ready",
                 4: "accumulator never drained", 5: "a peer's flag or counter never reached its value", 6: "internal hand-over"}


def _raise_status(v: int, device) -> None:
    status_word(device).zero_()
    raise RuntimeError(f"a device-side bounded wait ran out (status {v}: {_STATUS_NAMES.get(v, 'unknown')}); "
                       "the results of that step are incomplete; see csrc/ptx.cuh for codes")


def check_status(device: torch.device | None = None) -> int:
    """Synchronising read of the status word (call it between steps, not per kernel)."""
    v = int(status_word(device).item())
    if v != 0:
        _raise_status(v, device)
    return v


def set_wait_limit(seconds: float = 0.0) -> None:
    """Limit of every bounded device-side wait of the library on the current device (0 = the built-in 2 s).  Call it
    while no kernel of the library is running; tests use a few milliseconds to make a wait run out quickly."""
    raw = lib()._raw
    raw.csb_set_wait_ns.argtypes = [C.c_ulonglong]
    raw.csb_set_wait_ns.restype = C.c_int
    torch.cuda.synchronize()
    check(raw.csb_set_wait_ns(int(seconds * 1e9)), "csb_set_wait_ns")


_POLLS: dict[int, list] = {}


def poll_status(device: torch.device | None = None) -> None:
    """Check the status word WITHOUT synchronising: enqueue an asynchronous copy of it to pinned host memory and look
    at the copies enqueued by earlier calls whose events have completed.  Called once per step by the optimizer and the
    pipeline schedule, so a wait that ran out surfaces as an exception one step later at the latest (the optimizer has
    already skipped the update of the affected step on the device, see ``csb_clip_scale``).  Does nothing until a
    kernel with bounded waits has used the status word."""
    if not status_in_use(device):
        return
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    pending = _POLLS.setdefault(idx, [])
    while pending and pending[0][1].query():
        host, _ = pending.pop(0)
        v = int(host[0])
        if v != 0:
            pending.clear()
            _raise_status(v, device)
    if len(pending) < 4:
        host = torch.empty(1, dtype=torch.int32, pin_memory=True)
        host.copy_(_STATUS[idx], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        pending.append((host, ev))
