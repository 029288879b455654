"""Per-step training metrics as JSON lines: loss, tokens, device-timed step time (max over ranks), tokens/s.

The reference only prints a tqdm loss postfix on the last pipeline stage
(examples/distributed/run_vlm_hybrid.py:186-205) and has no throughput metric.  ``StepLogger`` times each step
with a CUDA event pair on the current stream (a host clock on CPU), reduces the time with MAX over the given
process group, and has rank 0 append one JSON object per step to a file (or stdout).
"""

from __future__ import annotations

import json
import sys
import time

import torch
import torch.distributed as dist


class StepLogger:
    def __init__(self, path: str | None = None, tokens_per_step: int = 0, group=None, extra: dict | None = None):
        self.path, self.tokens_per_step, self.group = path, tokens_per_step, group
        self.extra = extra or {}
        self.step = 0
        self._cuda = torch.cuda.is_available()
        self._t0 = None
        self.records: list[dict] = []
        self._fh = open(path, "a") if path and self._rank() == 0 else None

    def _rank(self) -> int:
        return dist.get_rank() if dist.is_initialized() else 0

    def begin(self):
        if self._cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.perf_counter()

    def end(self, loss=None, **fields) -> dict:
        if self._cuda:
            t1 = torch.cuda.Event(enable_timing=True)
            t1.record()
            t1.synchronize()
            ms = self._t0.elapsed_time(t1)
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            t = torch.tensor([ms], dtype=torch.float64, device="cuda" if (self._cuda and dist.get_backend(self.group) == "nccl") else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            ms = float(t.item())
        rec = {"step": self.step, "step_ms_max_over_ranks": round(ms, 3)}
        if loss is not None:
            rec["loss"] = float(loss)
        if self.tokens_per_step:
            rec["tokens"] = self.tokens_per_step
            rec["tokens_per_s"] = round(self.tokens_per_step / (ms / 1e3), 1)
        rec.update(self.extra)
        rec.update(fields)
        self.step += 1
        self.records.append(rec)
        if self._rank() == 0:
            line = json.dumps(rec)
            if self._fh is not None:
                self._fh.write(line + "\n")
                self._fh.flush()
            elif self.path is None:
                print(line, file=sys.stdout, flush=True)
        return rec

    def close(self):
        if self._fh is not None:
            self._fh.close()
            self._fh = None
