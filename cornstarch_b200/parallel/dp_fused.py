"""Data-parallel gradient reduction by a kernel of this package over NVLink peer memory (``csrc/grad_reduce.cu``).

The flat gradient buffers of :class:`cornstarch_b200.optim.fused_adamw.FusedAdamW` are allocated in peer-mapped
memory; one launch per buffer and rank then pulls the rank's slice from every peer, averages in fp32 and pushes the
bf16 result to every rank (all-reduce) or keeps it (reduce-scatter, for ZeRO-1).  The averaging scale and the cast
are part of the same pass, so a gradient element crosses HBM once on its owner and NVLink once per direction.

Stands in for the per-parameter ``all_reduce`` + ``div_`` loop of the reference
(cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:362-384).  Single node, 2..8 ranks,
bf16 gradients; everything else uses NCCL.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native as nat
from . import cp_fused  # noqa: F401  (declares csb_cp_signal / csb_cp_wait)
from .symm import SymmetricMemory

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_long, C.c_float
nat.declare("csb_grad_reduce", [vp, i32, i32, i64, f32, i32, vp, i32, i32, vp, vp])


class FusedGradReducer:
    _by_group: dict = {}

    @classmethod
    def get(cls, group) -> "FusedGradReducer | None":
        if group is None or not torch.cuda.is_available() or not dist.is_initialized() or dist.get_backend(group) != "nccl":
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > 8:
            return None
        if id(group) not in cls._by_group:
            cls._by_group[id(group)] = cls(group)
        return cls._by_group[id(group)]

    def __init__(self, group):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.flag_mem = SymmetricMemory(256, group)
        self.flags = self.flag_mem.local_tensor(torch.int32, 0, 64)
        self.flags.zero_()
        self.ready_ptrs = torch.tensor(list(self.flag_mem.ptrs), dtype=torch.int64, device="cuda")
        self.done_ptrs = torch.tensor([p + 128 for p in self.flag_mem.ptrs], dtype=torch.int64, device="cuda")
        self.events = 0
        self.buffers: list[tuple[SymmetricMemory, torch.Tensor]] = []
        torch.cuda.synchronize()
        dist.barrier(group)

    def allocate(self, numel: int, dtype=torch.bfloat16) -> torch.Tensor:
        """A zeroed flat buffer in peer-mapped memory (collective over the group: same sizes in the same order)."""
        assert dtype == torch.bfloat16 and numel % 8 == 0
        mem = SymmetricMemory(numel * 2, self.group)
        t = mem.local_tensor(torch.bfloat16, 0, numel)
        self.buffers.append((mem, t))
        return t

    def _find(self, t: torch.Tensor) -> SymmetricMemory:
        for mem, own in self.buffers:
            if own.data_ptr() == t.data_ptr():
                return mem
        raise KeyError("tensor was not allocated by this reducer")

    def reduce(self, tensors: list[torch.Tensor], scale: float | None = None, all_reduce: bool = True, max_ctas: int = 0):
        """Mean (``scale`` = 1/world by default) of every buffer over the group, in place.

        One counter exchange brackets all buffers: "my gradients are complete" before the first kernel, "my slices are
        pushed" after the last; the call returns (stream-ordered) once every rank's pushes have landed here."""
        lib, st = nat.lib(), nat.stream()
        status = nat.status_word(tensors[0].device)
        scale = 1.0 / self.world if scale is None else scale
        self.events += 1
        nat.check(lib.csb_cp_signal(self.ready_ptrs.data_ptr(), self.world, self.rank, self.events, st), "csb_cp_signal")
        for t in tensors:
            mem = self._find(t)
            nat.check(lib.csb_grad_reduce(C.cast(mem.ptr_array, vp), self.world, self.rank, t.numel(), scale, int(all_reduce),
                                          self.flags.data_ptr(), self.events, max_ctas, status.data_ptr(), st), "csb_grad_reduce")
        nat.check(lib.csb_cp_signal(self.done_ptrs.data_ptr(), self.world, self.rank, self.events, st), "csb_cp_signal")
        nat.check(lib.csb_cp_wait(self.flags.data_ptr() + 128, self.world, self.events, status.data_ptr(), st), "csb_cp_wait")
