"""``DcgmContextManager``: sample DCGM profiling fields (SM occupancy, tensor-pipe activity, SM activity,
framebuffer use) of this rank's GPU at 1 ms while a block runs.

Needs the DCGM host engine on ``localhost:5555`` and its Python bindings under
``/usr/local/dcgm/bindings/python3`` (as the reference aid, cornstarch/testing/dcgm.py:12-107).  When they
are absent, construction raises ``RuntimeError`` unless ``optional=True``, in which case the context is a
no-op and every trace is empty.  Nothing here changes a GPU setting.
"""

from __future__ import annotations

import os
import sys
import threading
import time
from contextlib import contextmanager

FIELDS = {"sm_occupancy": 1003, "tensor_active": 1004, "sm_active": 1002, "fb_used": 252}


class DcgmContextManager:
    def __init__(self, host: str = "localhost:5555", bindings: str = "/usr/local/dcgm/bindings/python3", optional: bool = False,
                 interval_us: int = 1000):
        self.available = False
        self.samples: dict[str, list[tuple[float, float]]] = {k: [] for k in FIELDS}
        self._stop = threading.Event()
        self._thread = None
        self.gpu = int(os.environ.get("LOCAL_RANK", "0"))
        self.interval_us = interval_us
        try:
            if bindings not in sys.path:
                sys.path.append(bindings)
            import pydcgm  # type: ignore
            import dcgm_fields  # type: ignore  # noqa: F401
            import dcgm_structs  # type: ignore

            self._pydcgm = pydcgm
            self._handle = pydcgm.DcgmHandle(ipAddress=host, opMode=dcgm_structs.DCGM_OPERATION_MODE_AUTO)
            self._group = pydcgm.DcgmGroup(self._handle, groupName=f"cornstarch_b200_{os.getpid()}", groupType=dcgm_structs.DCGM_GROUP_EMPTY)
            self._group.AddGpu(self.gpu)
            self._fields = pydcgm.DcgmFieldGroup(self._handle, name=f"csb_fields_{os.getpid()}", fieldIds=list(FIELDS.values()))
            self.available = True
        except Exception as e:  # noqa: BLE001
            if not optional:
                raise RuntimeError(f"DCGM is not available: {e}") from e

    def _poll(self):
        self._group.samples.WatchFields(self._fields, self.interval_us, 3600.0, 0)
        while not self._stop.is_set():
            vals = self._group.samples.GetLatest(self._fields).values
            now = time.time()
            for name, fid in FIELDS.items():
                try:
                    self.samples[name].append((now, vals[self.gpu][fid][-1].value))
                except Exception:  # noqa: BLE001
                    pass
            time.sleep(self.interval_us / 1e6)
        self._group.samples.UnwatchFields(self._fields)

    @contextmanager
    def profile(self):
        if not self.available:
            yield self
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()
        try:
            yield self
        finally:
            self._stop.set()
            self._thread.join()

    def get_sm_occupancy_trace(self):
        return self.samples["sm_occupancy"]

    def get_tensor_core_util_trace(self):
        return self.samples["tensor_active"]

    def get_sm_active_trace(self):
        return self.samples["sm_active"]

    def get_memory_usage_trace(self):
        return self.samples["fb_used"]
