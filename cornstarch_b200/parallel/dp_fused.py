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


class OverlappedGradReduce:
    """Reduce the gradients of a transformer layer as soon as the layer's backward pass has been enqueued, on a side
    stream with a few thread blocks, while the backward pass of the layers before it keeps the rest of the GPU busy.

    Used for the last micro-batch of a step (earlier micro-batches only accumulate).  The decoder loop announces every
    layer's input tensor through :func:`layer_input`; a hook on that tensor fires once the gradient with respect to it
    exists, i.e. after every backward node of the layer - and with it every weight-gradient kernel - has been issued.
    ``finish`` reduces what no hook covered (embeddings, head, encoders, norms outside the layers) and closes the
    exchange; after it the main stream sees averaged gradients everywhere.

    The reference reduces per parameter after the whole step
    (cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:362-384)."""

    current: "OverlappedGradReduce | None" = None

    def __init__(self, reducer: FusedGradReducer, flat_grads: list[torch.Tensor], max_ctas: int = 16):
        self.reducer, self.flat_grads, self.max_ctas = reducer, flat_grads, max_ctas
        self.side = torch.cuda.Stream()
        self.done: list[list[tuple[int, int]]] = [[] for _ in flat_grads]  # reduced element ranges per buffer
        self.launches = 0

    # ---- context: active while the last micro-batch runs forward and backward
    def __enter__(self):
        OverlappedGradReduce.current = self
        return self

    def __exit__(self, *exc):
        OverlappedGradReduce.current = None
        return False

    def _ranges_of(self, layer) -> list[tuple[int, int, int]]:
        cached = getattr(layer, "_csb_grad_ranges", None)
        if cached is not None:
            return cached
        spans: dict[int, list[int]] = {}
        for p in layer.parameters():
            g = getattr(p, "main_grad", None)
            if g is None:
                continue
            for bi, flat in enumerate(self.flat_grads):
                off = (g.data_ptr() - flat.data_ptr()) // flat.element_size()
                if 0 <= off < flat.numel() and g.data_ptr() >= flat.data_ptr():
                    lo = off // 64 * 64
                    hi = min(flat.numel(), (off + g.numel() + 63) // 64 * 64)
                    cur = spans.setdefault(bi, [lo, hi])
                    cur[0], cur[1] = min(cur[0], lo), max(cur[1], hi)
        out = [(bi, lo, hi) for bi, (lo, hi) in spans.items()]
        layer._csb_grad_ranges = out
        return out

    def layer_input(self, layer, tensor: torch.Tensor) -> None:
        if isinstance(tensor, torch.Tensor) and tensor.requires_grad:
            tensor.register_hook(lambda grad, layer=layer: self._layer_done(layer))

    def _layer_done(self, layer) -> None:
        ranges = [r for r in self._ranges_of(layer) if r[2] > r[1]]
        if not ranges:
            return
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            for bi, lo, hi in ranges:
                self._reduce_range(bi, lo, hi)

    def _reduce_range(self, bi: int, lo: int, hi: int) -> None:
        r = self.reducer
        lib, st = nat.lib(), nat.stream()
        flat = self.flat_grads[bi]
        mem = r._find(flat)
        status = nat.status_word(flat.device)
        r.events += 1
        nat.check(lib.csb_cp_signal(r.ready_ptrs.data_ptr(), r.world, r.rank, r.events, st), "csb_cp_signal")
        ptrs = (vp * 8)(*([p + lo * 2 for p in mem.ptrs] + [0] * (8 - r.world)))
        nat.check(lib.csb_grad_reduce(C.cast(ptrs, vp), r.world, r.rank, hi - lo, 1.0 / r.world, 1, r.flags.data_ptr(), r.events,
                                      self.max_ctas, status.data_ptr(), st), "csb_grad_reduce")
        self.done[bi].append((lo, hi))
        self.launches += 1

    @staticmethod
    def gaps(done: list[tuple[int, int]], numel: int) -> list[tuple[int, int]]:
        """The ranges of ``[0, numel)`` that no entry of ``done`` covers, in order."""
        out, pos = [], 0
        for lo, hi in sorted(done):
            if lo > pos:
                out.append((pos, lo))
            pos = max(pos, hi)
        if pos < numel:
            out.append((pos, numel))
        return out

    def finish(self, redo: list[tuple[int, int, int]] | None = None) -> None:
        """Reduce every range no layer hook covered, then wait until all ranks' pushes have landed here.

        ``redo``: ``(buffer, lo, hi)`` ranges that received a local contribution AFTER a hook may already have averaged
        them (gradients folded in from ``.grad``).  Such a range holds mean + local part; averaging it once more gives
        the full mean.  Ranges that fall into a gap are reduced once, by the gap."""
        r = self.reducer
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.side):
            self.side.wait_event(ev)
            saved, self.max_ctas = self.max_ctas, 0  # the backward pass is over: use the whole GPU
            for bi, flat in enumerate(self.flat_grads):
                gaps = self.gaps(self.done[bi], flat.numel())
                for lo, hi in gaps:
                    self._reduce_range(bi, lo, hi)
                for rb, lo, hi in redo or []:
                    if rb != bi:
                        continue
                    # the part of [lo, hi) that lies in hooked (already averaged) ranges
                    for dlo, dhi in self.gaps(gaps, flat.numel()):
                        a, b = max(lo, dlo), min(hi, dhi)
                        if a < b:
                            self._reduce_range(bi, a, b)
            self.max_ctas = saved
            lib, st = nat.lib(), nat.stream()
            status = nat.status_word(self.flat_grads[0].device)
            nat.check(lib.csb_cp_signal(r.done_ptrs.data_ptr(), r.world, r.rank, r.events, st), "csb_cp_signal")
            nat.check(lib.csb_cp_wait(r.flags.data_ptr() + 128, r.world, r.events, status.data_ptr(), st), "csb_cp_wait")
            end = torch.cuda.Event()
            end.record()
        torch.cuda.current_stream().wait_event(end)
        self.done = [[] for _ in self.flat_grads]


def layer_input(layer, tensor) -> None:
    """Called by a model's layer loop: lets an active :class:`OverlappedGradReduce` hook the layer's input."""
    cur = OverlappedGradReduce.current
    if cur is not None:
        cur.layer_input(layer, tensor)
