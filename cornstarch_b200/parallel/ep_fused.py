"""Expert-parallel dispatch / combine by this package's own kernel over NVLink peer memory (``csrc/moe_dispatch.cu``).

``FusedExpertExchange.exchange(src, index, counts)`` has the semantics of an uneven all-to-all: the rows this rank
sends are grouped by destination rank (``counts[me][d]`` rows for rank ``d``), the result holds the rows received,
grouped by source rank.  Instead of ``all_to_all_single`` every rank stores its rows straight into the receivers'
peer-mapped buffers; in the dispatch direction the gather of the tokens (``src[index]``) is part of the same copy.
Event counters order the three steps of a call: the slot is free (every peer has moved on from the call that used
it last), the rows have landed (every source has signalled), and receive buffers alternate between two slots.

The count matrix (rows from every source to every destination) is what the senders need to place their rows; it
comes from one small all-gather per MoE layer, which also yields the per-expert segment sizes on the receiver.
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native as nat
from . import cp_fused  # noqa: F401  (declares csb_cp_signal / csb_cp_wait)
from .symm import SymmetricMemory

vp, i32, i64 = C.c_void_p, C.c_int, C.c_long
nat.declare("csb_moe_push", [vp, vp, i64, i32, vp, vp, i32, i64, vp])
MAX = 8


class FusedExpertExchange:
    _by_group: dict = {}

    @classmethod
    def get(cls, group) -> "FusedExpertExchange | None":
        if group is None or not torch.cuda.is_available() or not dist.is_initialized() or dist.get_backend(group) != "nccl":
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > MAX:
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
        self.flag_ptrs = torch.tensor(list(self.flag_mem.ptrs), dtype=torch.int64, device="cuda")
        self.events = 0
        self.mem: SymmetricMemory | None = None
        self.capacity_rows = 0
        self.H = 0
        torch.cuda.synchronize()
        dist.barrier(group)

    def ensure(self, rows: int, H: int):
        """Two receive slots of ``rows`` rows each (collective; callers pass the same bound on every rank)."""
        if self.mem is not None and rows <= self.capacity_rows and H == self.H:
            return
        if self.mem is not None:
            self.mem.close()
        self.capacity_rows, self.H = rows, H
        self.mem = SymmetricMemory(2 * rows * H * 2, self.group)

    def exchange(self, src: torch.Tensor, index: torch.Tensor | None, counts: list[list[int]]) -> torch.Tensor:
        """``counts[s][d]`` = rows rank ``s`` sends to rank ``d``.  Returns the ``sum_s counts[s][me]`` received rows."""
        lib, st = nat.lib(), nat.stream()
        H = src.shape[1]
        me, ws = self.rank, self.world
        status = nat.status_word(src.device)
        slot = self.events % 2
        if self.events >= 2:
            # the slot was filled two calls ago; a peer has copied it out once it signalled the call after that one
            nat.check(lib.csb_cp_wait(self.flags.data_ptr(), ws, self.events, status.data_ptr(), st), "csb_cp_wait")
        seg = [0]
        for d in range(ws):
            seg.append(seg[-1] + counts[me][d])
        slot_bytes = self.capacity_rows * H * 2
        dst = []
        for d in range(ws):
            before = sum(counts[s][d] for s in range(me))  # rows of lower-ranked sources come first in d's buffer
            assert before + counts[me][d] <= self.capacity_rows, "receive buffer too small"
            dst.append(self.mem.ptrs[d] + slot * slot_bytes + before * H * 2)
        seg_arr = (i32 * (ws + 1))(*seg)
        dst_arr = (vp * ws)(*dst)
        idx = index.int().contiguous() if index is not None else None
        srcc = src.contiguous()
        nat.check(lib.csb_moe_push(srcc.data_ptr(), nat.ptr(idx), seg[-1], H, C.cast(seg_arr, vp), C.cast(dst_arr, vp), ws, srcc.shape[0], st), "csb_moe_push")
        self.events += 1
        nat.check(lib.csb_cp_signal(self.flag_ptrs.data_ptr(), ws, me, self.events, st), "csb_cp_signal")
        nat.check(lib.csb_cp_wait(self.flags.data_ptr(), ws, self.events, status.data_ptr(), st), "csb_cp_wait")
        n_recv = sum(counts[s][me] for s in range(ws))
        buf = self.mem.local_tensor(torch.bfloat16, slot * slot_bytes, n_recv * H).view(n_recv, H)
        return buf.clone()  # the slot is reused two calls later


class _FusedA2A(torch.autograd.Function):
    """Uneven all-to-all through peer memory; the backward is the reverse exchange (and the scatter-add of a fused gather)."""

    @staticmethod
    def forward(ctx, x, index, counts, ex: FusedExpertExchange):
        ctx.ex, ctx.counts, ctx.n_src = ex, counts, x.shape[0]
        ctx.save_for_backward(index) if index is not None else ctx.save_for_backward()
        ctx.has_index = index is not None
        return ex.exchange(x, index, counts)

    @staticmethod
    def backward(ctx, g):
        ws = ctx.ex.world
        rev = [[ctx.counts[d][s] for d in range(ws)] for s in range(ws)]
        back = ctx.ex.exchange(g.contiguous(), None, rev)  # rows in this rank's original send order
        if ctx.has_index:
            (index,) = ctx.saved_tensors
            gx = torch.zeros((ctx.n_src, g.shape[1]), dtype=g.dtype, device=g.device)
            gx.index_add_(0, index.long(), back)
            return gx, None, None, None
        return back, None, None, None


def fused_all_to_all(x, index, counts, ex):
    return _FusedA2A.apply(x, index, counts, ex)
