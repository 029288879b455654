"""Context-parallel attention fused with its collectives over NVLink peer memory.

The reference gathers K and V with NCCL before every attention call and reduce-scatters dK / dV after the backward
(cornstarch/shardformer/layers/context_parallel_bitfield_attention.py:66-135 forward all-gather per head stride,
:183-318 backward all-gather + two reduce-scatters).  Here nothing is gathered:

* forward: every rank copies its K / V shard into a peer-mapped staging buffer and bumps a counter in every peer's
  flag array.  The flash-attention kernel receives one tensor map per rank ("segments") and streams key / value
  tiles straight out of the owning GPU's memory with plain (non-multicast) TMA loads, tile by tile under the same
  tile-class skip list as the local kernel.  Tiles of the rank's own shard come first, so the (bounded) wait for a
  peer's counter is hidden behind local work.
* backward: the key-stationary kernel loads each key block from its owner the same way and writes the block's
  dK / dV tile into the owner's inbox slot of this rank; after a second counter exchange each owner sums its
  ``world`` inbox slots (fp32 accumulation).  This is the reduce-scatter, done by the kernels themselves.

Staging buffers alternate between two slots, which together with the counters is enough: a rank that has seen all
counters of call ``n+1`` knows every peer has finished reading the buffers of call ``n``.

Every rank must issue the same sequence of calls (same layers, same order, forward and backward), which is what
data / context parallel training does.  Single node, world size 2..8, bf16.
"""

from __future__ import annotations

import ctypes as C
import math
import os

import torch
import torch.distributed as dist

from ..ops import _native as nat
from ..ops import attention as A
from .symm import SymmetricMemory

MAX_SEG = 8
vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_long, C.c_float


class KvSegments(C.Structure):
    """Mirror of ``CsbKvSegments`` (csrc/kv_segments.h)."""

    _fields_ = [
        ("n_seg", i32), ("my_seg", i32), ("rows", i32 * MAX_SEG),
        ("k", vp * MAX_SEG), ("v", vp * MAX_SEG),
        ("k_stride_s", i64 * MAX_SEG), ("k_stride_b", i64 * MAX_SEG),
        ("v_stride_s", i64 * MAX_SEG), ("v_stride_b", i64 * MAX_SEG),
        ("ready_flags", vp), ("ready_value", i32),
        ("dk", vp * MAX_SEG), ("dv", vp * MAX_SEG),
        ("dk_stride_s", i64 * MAX_SEG), ("dk_stride_b", i64 * MAX_SEG),
        ("dv_stride_s", i64 * MAX_SEG), ("dv_stride_b", i64 * MAX_SEG),
        ("pull_ctas", i32), ("pull_k", vp * MAX_SEG), ("pull_v", vp * MAX_SEG), ("pull_elems", i64 * MAX_SEG),
        ("pulled", vp), ("pull_target", i32),
    ]


nat.declare("csb_attn_fwd_seg", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, f32, i32, vp, vp, vp, vp, vp, vp, vp])
nat.declare("csb_attn_bwd_seg", [vp, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64,
                                 i64, i64, f32, i32, vp, vp, vp, vp, vp, vp, vp])
nat.declare("csb_cp_signal", [vp, i32, i32, i32, vp])
nat.declare("csb_cp_reduce", [vp, i32, vp, i32, vp, i64, vp, vp])
nat.declare("csb_cp_wait", [vp, i32, i32, vp, vp])


# thread blocks of the forward kernel that copy remote K / V into local memory (0: every tile is read from its owner)
PULL_CTAS = int(os.environ.get("CORNSTARCH_B200_CP_PULL_CTAS", "24"))


def padded_layout(sizes: list[int], tile: int = 128):
    """Start of every rank's segment in the padded gathered index space, and its total length."""
    starts, n = [], 0
    for s in sizes:
        starts.append(n)
        n += (s + tile - 1) // tile * tile
    return starts, n


class _Buffers:
    """Peer-mapped memory for one (batch, max shard length, kv heads, head dim) shape."""

    def __init__(self, group, B: int, smax: int, Hk: int, D: int):
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.B, self.smax, self.Hk, self.D = B, smax, Hk, D
        self.slot = B * smax * Hk * D * 2  # bytes of one [B][smax][Hk][D] bf16 tensor
        self.off_kv = 0                               # 2 buffers x (K, V)
        self.off_inbox = 4 * self.slot                # world source ranks x (dK, dV)
        self.off_flags = self.off_inbox + 2 * self.world * self.slot
        total = self.off_flags + 2 * 128
        self.mem = SymmetricMemory(total, group)
        flags = self.mem.local_tensor(torch.int32, self.off_flags, 64)
        flags.zero_()
        self.flags = flags
        # device arrays of the peers' flag-array addresses (kv-ready flags, dkv-delivered flags)
        self.kv_flag_ptrs = torch.tensor([p + self.off_flags for p in self.mem.ptrs], dtype=torch.int64, device="cuda")
        self.dkv_flag_ptrs = torch.tensor([p + self.off_flags + 128 for p in self.mem.ptrs], dtype=torch.int64, device="cuda")
        self.kv_events = 0
        self.dkv_events = 0
        # forward: local copies of the peers' K / V (filled by the kernel's pulling blocks) and their completion counters
        self.pull = torch.empty((self.world, 2, B, smax, Hk, D), dtype=torch.bfloat16, device="cuda")
        self.pulled = torch.zeros(MAX_SEG, dtype=torch.int32, device="cuda")
        self.pull_calls = 0
        torch.cuda.synchronize()
        dist.barrier(group)

    def shape(self):
        return (self.B, self.smax, self.Hk, self.D)

    def local(self, offset: int) -> torch.Tensor:
        return self.mem.local_tensor(torch.bfloat16, offset, self.slot // 2).view(self.B, self.smax, self.Hk, self.D)


class FusedContextParallelAttention:
    """Per process group: staging / inbox buffers and the event counters of the fused context-parallel attention."""

    _by_group: dict = {}

    @classmethod
    def get(cls, group) -> "FusedContextParallelAttention | None":
        if group is None or not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > MAX_SEG:
            return None
        if id(group) not in cls._by_group:
            cls._by_group[id(group)] = cls(group)
        return cls._by_group[id(group)]

    def __init__(self, group):
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self._bufs: dict = {}

    def buffers(self, B, smax, Hk, D) -> _Buffers:
        key = (B, smax, Hk, D)
        if key not in self._bufs:
            self._bufs[key] = _Buffers(self.group, B, smax, Hk, D)
        return self._bufs[key]

    # ------------------------------------------------------------------ building blocks
    def stage_kv(self, bufs: _Buffers, k: torch.Tensor, v: torch.Tensor):
        """Copy this rank's K / V shard into the staging slot of this call and publish the new counter to all peers."""
        which = bufs.kv_events % 2
        S = k.shape[1]
        if bufs.kv_events >= 2:
            # the slot was last used two calls ago: every peer must have finished that call's kernels, which it has once
            # it staged the call after it (a kernel only waits for the peers whose tiles its mask needs, so this
            # explicit wait is what covers the others)
            st = nat.status_word(k.device)
            nat.check(nat.lib().csb_cp_wait(bufs.flags.data_ptr(), self.world, bufs.kv_events, st.data_ptr(), nat.stream()),
                      "csb_cp_wait")
        bufs.local(bufs.off_kv + (2 * which) * bufs.slot)[:, :S].copy_(k)
        bufs.local(bufs.off_kv + (2 * which + 1) * bufs.slot)[:, :S].copy_(v)
        bufs.kv_events += 1
        nat.check(nat.lib().csb_cp_signal(bufs.kv_flag_ptrs.data_ptr(), self.world, self.rank, bufs.kv_events, nat.stream()),
                  "csb_cp_signal")
        return which, bufs.kv_events

    def segments(self, bufs: _Buffers, sizes: list[int], which: int, value: int, with_grads: bool) -> KvSegments:
        seg = KvSegments()
        seg.n_seg, seg.my_seg = self.world, self.rank
        ss, sb = bufs.Hk * bufs.D, bufs.smax * bufs.Hk * bufs.D
        for r in range(self.world):
            base = bufs.mem.ptrs[r]
            seg.rows[r] = sizes[r]
            seg.k[r] = base + bufs.off_kv + (2 * which) * bufs.slot
            seg.v[r] = base + bufs.off_kv + (2 * which + 1) * bufs.slot
            seg.k_stride_s[r] = seg.v_stride_s[r] = ss
            seg.k_stride_b[r] = seg.v_stride_b[r] = sb
            if with_grads:
                # rank r's inbox, slot of this (source) rank
                seg.dk[r] = base + bufs.off_inbox + (2 * self.rank) * bufs.slot
                seg.dv[r] = base + bufs.off_inbox + (2 * self.rank + 1) * bufs.slot
                seg.dk_stride_s[r] = seg.dv_stride_s[r] = ss
                seg.dk_stride_b[r] = seg.dv_stride_b[r] = sb
        seg.ready_flags = bufs.flags.data_ptr()
        seg.ready_value = value
        if not with_grads and PULL_CTAS > 0:
            # forward: a query tile needs most key tiles, so remote K / V are copied once into local memory by the
            # first thread blocks of the kernel instead of being fetched over NVLink by every query tile
            bufs.pull_calls += 1
            seg.pull_ctas = PULL_CTAS
            seg.pulled = bufs.pulled.data_ptr()
            seg.pull_target = PULL_CTAS * bufs.pull_calls
            for r in range(self.world):
                seg.pull_k[r] = bufs.pull[r, 0].data_ptr()
                seg.pull_v[r] = bufs.pull[r, 1].data_ptr()
                seg.pull_elems[r] = (sizes[r] if bufs.B == 1 else bufs.smax) * bufs.B * bufs.Hk * bufs.D
        return seg

    # ------------------------------------------------------------------ forward / backward
    def forward(self, q, k, v, sizes: list[int], mask: A.AttnMask, scale):
        B, Sq, Hq, D = q.shape
        Hk = k.shape[2]
        bufs = self.buffers(B, max(sizes), Hk, D)
        which, value = self.stage_kv(bufs, k, v)
        seg = self.segments(bufs, sizes, which, value, with_grads=False)
        _, Sk = padded_layout(sizes)
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        q = q if (q.stride(3) == 1 and q.stride(2) == D and q.stride(1) % 8 == 0) else q.contiguous()
        out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
        cls = mask.classes(B, Sq, Sk, q.device)
        qb, kb, qp, kp = A._mask_ptrs(mask, B)
        st = nat.status_word(q.device)
        nat.check(nat.lib().csb_attn_fwd_seg(
            q.data_ptr(), C.addressof(seg), out.data_ptr(), lse.data_ptr(), B, Sq, Sk, Hq, Hk, D, q.stride(1), q.stride(0),
            out.stride(1), out.stride(0), scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp),
            cls.data_ptr(), st.data_ptr(), nat.stream()), "csb_attn_fwd_seg")
        return out, lse

    def backward(self, do, q, k, v, out, lse, sizes: list[int], mask: A.AttnMask, scale):
        B, Sq, Hq, D = q.shape
        Hk = k.shape[2]
        bufs = self.buffers(B, max(sizes), Hk, D)
        which, value = self.stage_kv(bufs, k, v)  # the peers read this rank's K / V again
        seg = self.segments(bufs, sizes, which, value, with_grads=True)
        _, Sk = padded_layout(sizes)
        scale = scale if scale is not None else 1.0 / math.sqrt(D)
        if do.stride(3) != 1 or do.stride(2) != D or do.stride(1) % 8:
            do = do.contiguous()
        q = q if (q.stride(3) == 1 and q.stride(2) == D and q.stride(1) % 8 == 0) else q.contiguous()
        dq = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
        dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
        delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
        cls = mask.classes(B, Sq, Sk, q.device)
        qb, kb, qp, kp = A._mask_ptrs(mask, B)
        st = nat.status_word(q.device)
        nat.check(nat.lib().csb_attn_bwd_seg(
            q.data_ptr(), C.addressof(seg), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
            dq.data_ptr(), B, Sq, Sk, Hq, Hk, D, q.stride(1), q.stride(0), out.stride(1), out.stride(0), do.stride(1),
            do.stride(0), dq.stride(1), dq.stride(0), scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp),
            cls.data_ptr(), st.data_ptr(), nat.stream()), "csb_attn_bwd_seg")
        # every dK / dV tile of this rank has been written into its owner's inbox: tell the owners, then sum my inbox
        bufs.dkv_events += 1
        nat.check(nat.lib().csb_cp_signal(bufs.dkv_flag_ptrs.data_ptr(), self.world, self.rank, bufs.dkv_events, nat.stream()),
                  "csb_cp_signal")
        n = bufs.slot // 2
        outs = []
        for which_grad in (0, 1):
            src = (vp * MAX_SEG)(*[bufs.mem.ptrs[self.rank] + bufs.off_inbox + (2 * r + which_grad) * bufs.slot
                                   for r in range(self.world)] + [0] * (MAX_SEG - self.world))
            res = torch.empty((B, bufs.smax, Hk, D), dtype=q.dtype, device=q.device)
            nat.check(nat.lib().csb_cp_reduce(C.cast(src, vp), self.world, bufs.flags.data_ptr() + 128, bufs.dkv_events,
                                              res.data_ptr(), n, st.data_ptr(), nat.stream()), "csb_cp_reduce")
            outs.append(res[:, : k.shape[1]])
        return dq, outs[0], outs[1]


class _FusedCpAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, fused, sizes, mask, scale):
        out, lse = fused.forward(q, k, v, sizes, mask, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.fused, ctx.sizes, ctx.mask, ctx.scale = fused, sizes, mask, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ctx.fused.backward(do, q, k, v, out, lse, ctx.sizes, ctx.mask, ctx.scale)
        return dq, dk, dv, None, None, None, None


class _FusedCpAttnReplayFn(torch.autograd.Function):
    """Forward output kept across an activation recomputation; backward runs the fused kernels."""

    @staticmethod
    def forward(ctx, q, k, v, fused, sizes, mask, scale, out, lse):
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.fused, ctx.sizes, ctx.mask, ctx.scale = fused, sizes, mask, scale
        return out.view_as(out)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ctx.fused.backward(do, q, k, v, out, lse, ctx.sizes, ctx.mask, ctx.scale)
        return dq, dk, dv, None, None, None, None, None, None


def padded_mask(local_mask: A.AttnMask, sizes: list[int]) -> A.AttnMask:
    """The mask of the local queries against the gathered keys, re-indexed to the padded gathered space
    (pad entries: position -1, bits 0, i.e. never attended)."""
    starts, total = padded_layout(sizes)
    kp, kb = local_mask.k_pos, local_mask.k_bits
    B = kp.shape[0]
    dev = kp.device
    idx = torch.cat([torch.arange(s, s + n, device=dev) for s, n in zip(starts, sizes)])
    new_kp = torch.full((B, total), -1, dtype=torch.int32, device=dev)
    new_kp[:, idx] = kp.int()
    new_kb = None
    if kb is not None:
        new_kb = torch.zeros((B, total), dtype=torch.int64, device=dev)
        new_kb[:, idx] = kb
    return A.AttnMask(mode=local_mask.mode, q_bits=local_mask.q_bits, k_bits=new_kb, q_pos=local_mask.q_pos, k_pos=new_kp)


def fused_context_parallel_attention(q, k, v, fused: FusedContextParallelAttention, sizes: list[int], mask: A.AttnMask, scale=None):
    """Local queries against all ranks' keys / values (``mask`` in the padded gathered index space)."""
    tape = getattr(A._TAPE, "cur", None)
    if tape is not None and tape.mode == "record" and not torch.is_grad_enabled():
        out, lse = fused.forward(q, k, v, sizes, mask, scale)
        tape.items.append((out, lse))
        return out
    if tape is not None and tape.mode == "replay" and tape.items:
        out, lse = tape.items.pop(0)
        return _FusedCpAttnReplayFn.apply(q, k, v, fused, sizes, mask, scale, out, lse)
    return _FusedCpAttnFn.apply(q, k, v, fused, sizes, mask, scale)


def local_segments(ks: list[torch.Tensor], vs: list[torch.Tensor], my_seg: int = 0, dks=None, dvs=None) -> KvSegments:
    """Segments that all live in this GPU's memory (no flags): the kernels' segment logic without any peer."""
    seg = KvSegments()
    seg.n_seg, seg.my_seg = len(ks), my_seg
    for r, (k, v) in enumerate(zip(ks, vs)):
        seg.rows[r] = k.shape[1]
        seg.k[r], seg.v[r] = k.data_ptr(), v.data_ptr()
        seg.k_stride_s[r], seg.k_stride_b[r] = k.stride(1), k.stride(0)
        seg.v_stride_s[r], seg.v_stride_b[r] = v.stride(1), v.stride(0)
        if dks is not None:
            seg.dk[r], seg.dv[r] = dks[r].data_ptr(), dvs[r].data_ptr()
            seg.dk_stride_s[r], seg.dk_stride_b[r] = dks[r].stride(1), dks[r].stride(0)
            seg.dv_stride_s[r], seg.dv_stride_b[r] = dvs[r].stride(1), dvs[r].stride(0)
    seg.ready_flags = None
    seg.ready_value = 0
    return seg


def attention_segments_local(q, ks, vs, mask: A.AttnMask, scale=None, my_seg: int = 0, do=None, pull_ctas: int = 0):
    """Forward (and backward when ``do`` is given) over K/V given as several local tensors; ``mask`` is indexed in the
    padded gathered space of ``[k.shape[1] for k in ks]``.  Returns ``(out, lse)`` or ``(out, lse, dq, dks, dvs)``.

    ``pull_ctas > 0`` runs the forward the way the multi-GPU path does: the first thread blocks copy every segment but
    ``my_seg`` into a second buffer (the ready counters are already set) and the query tiles read those copies."""
    B, Sq, Hq, D = q.shape
    Hk = ks[0].shape[2]
    sizes = [k.shape[1] for k in ks]
    _, Sk = padded_layout(sizes)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    cls = mask.classes(B, Sq, Sk, q.device)
    qb, kb, qp, kp = A._mask_ptrs(mask, B)
    st = nat.status_word(q.device)
    seg = local_segments(ks, vs, my_seg)
    if pull_ctas > 0:
        assert all(k.is_contiguous() and v.is_contiguous() for k, v in zip(ks, vs))
        keep = [torch.ones(MAX_SEG, dtype=torch.int32, device=q.device), torch.zeros(MAX_SEG, dtype=torch.int32, device=q.device)]
        seg.ready_flags, seg.ready_value = keep[0].data_ptr(), 1
        seg.pull_ctas, seg.pulled, seg.pull_target = pull_ctas, keep[1].data_ptr(), pull_ctas
        for r, (k, v) in enumerate(zip(ks, vs)):
            ck, cv = torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
            keep += [ck, cv]
            seg.pull_k[r], seg.pull_v[r], seg.pull_elems[r] = ck.data_ptr(), cv.data_ptr(), k.numel()
    nat.check(nat.lib().csb_attn_fwd_seg(
        q.data_ptr(), C.addressof(seg), out.data_ptr(), lse.data_ptr(), B, Sq, Sk, Hq, Hk, D, q.stride(1), q.stride(0),
        out.stride(1), out.stride(0), scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp), cls.data_ptr(),
        st.data_ptr(), nat.stream()), "csb_attn_fwd_seg")
    if do is None:
        return out, lse
    dks = [torch.empty_like(k) for k in ks]
    dvs = [torch.empty_like(v) for v in vs]
    seg = local_segments(ks, vs, my_seg, dks, dvs)
    dq = torch.empty_like(q)
    dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    nat.check(nat.lib().csb_attn_bwd_seg(
        q.data_ptr(), C.addressof(seg), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(),
        dq.data_ptr(), B, Sq, Sk, Hq, Hk, D, q.stride(1), q.stride(0), out.stride(1), out.stride(0), do.stride(1),
        do.stride(0), dq.stride(1), dq.stride(0), scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp),
        cls.data_ptr(), st.data_ptr(), nat.stream()), "csb_attn_bwd_seg")
    return out, lse, dq, dks, dvs
