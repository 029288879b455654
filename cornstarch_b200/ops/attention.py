"""Bitfield / causal / full flash attention (forward + backward) on the tcgen05 kernels.

Public pieces:

* :class:`AttnMask` — what the kernels need to know about the mask: a mode, optional int64 bitfields
  for queries and keys, optional explicit token positions (context parallelism hands each rank a
  non-contiguous token set) and the cached tile-class map.
* :func:`dense_mask` — boolean ``[B, Sq, Sk]`` statement of the predicate (oracle, CPU path).
* :func:`attention` — autograd-aware ``softmax(scale q k^T + mask) v`` for ``[B, S, H, D]`` tensors with GQA.

Mask semantics follow the reference kernel (cornstarch/kernel/bitfield_attention.py:86-101); see
``csrc/mask.cuh``.  The kernels replace cornstarch/kernel/bitfield_attention.py (T4-T9) and
cornstarch/kernel/attention.py (T1-T3), and the FA2 calls of
cornstarch/shardformer/layers/context_parallel_attention.py.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import threading

import torch
import torch.nn.functional as F

from . import _native as nat

MASK_FULL, MASK_CAUSAL, MASK_BITFIELD, MASK_BITFIELD_PREFIX_CAUSAL, MASK_DENSE = 0, 1, 2, 3, 4
_LOW62 = (1 << 62) - 1
BLOCK = 128

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_long, C.c_float
nat.declare("csb_mask_classify", [i32, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp])
nat.declare(
    "csb_attn_fwd",
    [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i64, i64, i64, i64, i64, i64, i64, i64, f32, i32, vp, vp, vp, vp,
     vp, vp, vp],
)
nat.declare(
    "csb_attn_bwd",
    [vp] * 11 + [i32] * 6 + [i64] * 16 + [f32, i32, vp, vp, vp, vp, vp, vp, vp],
)
nat.declare("csb_mask_classify_dense", [vp, i64, i64, i32, i32, i32, vp, vp, vp])
nat.declare("csb_attn_fwd_dense", [vp] * 5 + [i32] * 6 + [i64] * 8 + [f32, i32, vp, vp, vp, vp])
nat.declare("csb_attn_bwd_dense", [vp] * 11 + [i32] * 6 + [i64] * 16 + [f32, i32, vp, vp, vp, vp])


class _Extras(C.Structure):
    """``CsbAttnExtras`` of the native library: dense boolean mask and additive bias of one attention call."""

    _fields_ = [("dmask", vp), ("dm_sb", i64), ("dm_sq", i64), ("bias", vp), ("bias_sb", i64), ("bias_sh", i64), ("bias_sq", i64)]


@dataclass
class AttnMask:
    """Mask description shared by every layer of a forward/backward pass."""

    mode: int = MASK_CAUSAL
    q_bits: torch.Tensor | None = None  # int64 [B, Sq]
    k_bits: torch.Tensor | None = None  # int64 [B, Sk]
    q_pos: torch.Tensor | None = None  # int32 [B, Sq] global positions of the local query rows
    k_pos: torch.Tensor | None = None  # int32 [B, Sk]
    dense: torch.Tensor | None = None  # bool / uint8 [B, Sq, Sk] (True = attend), mode MASK_DENSE
    bias: torch.Tensor | None = None  # additive, broadcastable to [B, H, Sq, Sk] (no gradient), with MASK_FULL or MASK_DENSE
    _cls: dict = field(default_factory=dict, repr=False)

    @staticmethod
    def full() -> "AttnMask":
        return AttnMask(mode=MASK_FULL)

    @staticmethod
    def causal() -> "AttnMask":
        return AttnMask(mode=MASK_CAUSAL)

    @staticmethod
    def bitfield(bits: torch.Tensor, k_bits: torch.Tensor | None = None, prefix_causal: bool = False,
                 q_pos: torch.Tensor | None = None, k_pos: torch.Tensor | None = None) -> "AttnMask":
        return AttnMask(
            mode=MASK_BITFIELD_PREFIX_CAUSAL if prefix_causal else MASK_BITFIELD,
            q_bits=bits, k_bits=bits if k_bits is None else k_bits, q_pos=q_pos, k_pos=k_pos,
        )

    @staticmethod
    def from_dense(mask: torch.Tensor | None, bias: torch.Tensor | None = None) -> "AttnMask":
        """Flash attention with a dense boolean mask ``[B, Sq, Sk]`` and / or an additive bias (the reference's
        ``flash_attn_func(q, k, v, bias, mask)``, cornstarch/kernel/attention.py:1126-1147)."""
        if mask is None:
            return AttnMask(mode=MASK_FULL, bias=bias)
        if mask.dim() == 4:
            assert mask.shape[1] == 1, "a dense mask is shared by all heads"
            mask = mask[:, 0]
        return AttnMask(mode=MASK_DENSE, dense=mask, bias=bias)

    def extras(self, B: int, H: int, Sq: int, Sk: int, device, with_bias: bool = True):
        """ctypes ``CsbAttnExtras`` (plus the tensors it points to, which the caller keeps alive) or ``(None, ())``."""
        if self.dense is None and (self.bias is None or not with_bias):
            return None, ()
        keep = []
        ex = _Extras()
        if self.dense is not None:
            m = self._cls.get("dense_u8")
            if m is None:
                m = self.dense.to(device=device).ne(0).to(torch.uint8)
                if m.shape[0] == 1 and B > 1:
                    m = m.expand(B, -1, -1)
                m = m.contiguous()
                self._cls["dense_u8"] = m
            assert m.shape == (B, Sq, Sk), f"dense mask {tuple(m.shape)} does not match {(B, Sq, Sk)}"
            ex.dmask, ex.dm_sb, ex.dm_sq = m.data_ptr(), m.stride(0), m.stride(1)
            keep.append(m)
        if self.bias is not None and with_bias:
            bz = self._cls.get("bias_f32")
            if bz is None:
                bz = self.bias.to(device=device, dtype=torch.float32)
                while bz.dim() < 4:
                    bz = bz.unsqueeze(0)
                if bz.stride(-1) != 1:
                    bz = bz.contiguous()
                self._cls["bias_f32"] = bz
            e = bz.expand(B, H, Sq, Sk)
            ex.bias, ex.bias_sb, ex.bias_sh, ex.bias_sq = bz.data_ptr(), e.stride(0), e.stride(1), e.stride(2)
            keep.append(bz)
        return ex, tuple(keep)

    def classes(self, B: int, Sq: int, Sk: int, device) -> torch.Tensor:
        """int8 ``[B, nQ, nK]`` tile classes for 128x128 tiles (0 skip, 1 mixed, 2 all allowed); cached."""
        key = (B, Sq, Sk, str(device))
        c = self._cls.get(key)
        if c is None:
            c = classify_mask(self, B, Sq, Sk, device)
            self._cls[key] = c
        return c


def dense_mask(mask: AttnMask, B: int, Sq: int, Sk: int, device="cpu") -> torch.Tensor:
    """Boolean ``[B, Sq, Sk]`` (True = may attend): direct statement of the per-element predicate."""
    qp = mask.q_pos.to(device).long() if mask.q_pos is not None else torch.arange(Sq, device=device).expand(B, Sq)
    kp = mask.k_pos.to(device).long() if mask.k_pos is not None else torch.arange(Sk, device=device).expand(B, Sk)
    qp, kp = qp[:, :, None], kp[:, None, :]
    if mask.mode == MASK_FULL:
        return torch.ones(B, Sq, Sk, dtype=torch.bool, device=device)
    if mask.mode == MASK_DENSE:
        return mask.dense.to(device).ne(0).expand(B, Sq, Sk)
    if mask.mode == MASK_CAUSAL:
        return (kp <= qp).expand(B, Sq, Sk).clone()
    qb = (mask.q_bits.to(device) & _LOW62)[:, :, None]
    kb = (mask.k_bits.to(device) & _LOW62)[:, None, :]
    nonpad = (qb != 0) & (kb != 0)
    q_text = (qb & 1) != 0
    text_rule = q_text & (kp <= qp) & ((qb & kb) != 0)
    modal_rule = (~q_text) & (qb == kb)
    if mask.mode == MASK_BITFIELD_PREFIX_CAUSAL:
        modal_rule = modal_rule | ((~q_text) & (kp < qp))
    return nonpad & (text_rule | modal_rule)


def classify_mask(mask: AttnMask, B: int, Sq: int, Sk: int, device, bm: int = BLOCK, bn: int = BLOCK,
                  with_work: bool = False):
    """Tile classes of the mask; on CUDA by the native kernel, otherwise from the dense predicate."""
    nQ, nK = (Sq + bm - 1) // bm, (Sk + bn - 1) // bn
    dev = torch.device(device)
    if dev.type != "cuda":
        d = dense_mask(mask, B, Sq, Sk, dev)
        pad = torch.zeros(B, nQ * bm, nK * bn, dtype=torch.bool, device=dev)
        pad[:, :Sq, :Sk] = d
        cnt = pad.view(B, nQ, bm, nK, bn).sum(dim=(2, 4))
        rows = torch.clamp(Sq - torch.arange(nQ, device=dev) * bm, max=bm)[None, :, None]
        cls = torch.ones(B, nQ, nK, dtype=torch.int8, device=dev)
        cls[cnt == 0] = 0
        cls[cnt == rows * bn] = 2
        if with_work:
            return cls, (cls != 0).sum(-1).int()
        return cls
    cls = torch.empty(B, nQ, nK, dtype=torch.int8, device=dev)
    work = torch.zeros(B, nQ, dtype=torch.int32, device=dev) if with_work else None
    if mask.mode == MASK_DENSE:
        assert bm == BLOCK and bn == BLOCK, "dense masks are classified in 128 x 128 tiles"
        ex, keep = mask.extras(B, 1, Sq, Sk, dev, with_bias=False)
        nat.check(nat.lib().csb_mask_classify_dense(ex.dmask, ex.dm_sb, ex.dm_sq, B, Sq, Sk, cls.data_ptr(), nat.ptr(work),
                                                    nat.stream()), "csb_mask_classify_dense")
        return (cls, work) if with_work else cls
    qb, kb, qp, kp = _mask_ptrs(mask, B)
    nat.check(
        nat.lib().csb_mask_classify(mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp), B, Sq, Sk, bm, bn,
                                    cls.data_ptr(), nat.ptr(work), nat.stream()),
        "csb_mask_classify",
    )
    return (cls, work) if with_work else cls


def attention_reference(q, k, v, mask: AttnMask, scale: float | None = None):
    """fp32 PyTorch attention with the dense mask; fully masked rows give 0 (and LSE = -inf)."""
    B, Sq, Hq, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    g = Hq // Hk
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask.bias is not None:
        s = s + mask.bias.to(device=q.device, dtype=torch.float32)
    m = dense_mask(mask, B, Sq, Sk, q.device)[:, None]
    s = s.masked_fill(~m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    p = torch.where(m, p, torch.zeros_like(p))
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def _check_layout(t: torch.Tensor, name: str):
    assert t.dim() == 4 and t.stride(3) == 1 and t.stride(2) == t.shape[3], f"{name} must be [B,S,H,D] with dense heads"
    assert t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0, f"{name}: token stride / base must be 16-byte aligned"


def _rows(t, B, to_int=False):
    """Per-token mask metadata as a contiguous ``[B, S]`` tensor (a single row is shared by the whole batch)."""
    if t is None:
        return None
    if to_int:
        t = t.int()
    if B is not None and t.shape[0] == 1 and B > 1:
        t = t.expand(B, -1)
    return t.contiguous()


def _mask_ptrs(mask: AttnMask, B: int | None = None):
    return _rows(mask.q_bits, B), _rows(mask.k_bits, B), _rows(mask.q_pos, B, True), _rows(mask.k_pos, B, True)


def attention_forward(q, k, v, mask: AttnMask, scale: float | None = None):
    """Native forward; returns ``(out [B,Sq,Hq,D] bf16, lse [B,Hq,Sq] fp32)``."""
    B, Sq, Hq, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _check_layout(t, n)
    out = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    cls = mask.classes(B, Sq, Sk, q.device)
    st = nat.status_word(q.device)
    ex, keep = mask.extras(B, Hq, Sq, Sk, q.device)
    if ex is not None:
        nat.check(
            nat.lib().csb_attn_fwd_dense(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, Sq, Sk, Hq, Hk, D,
                q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0), out.stride(1), out.stride(0),
                scale, mask.mode, cls.data_ptr(), C.addressof(ex), st.data_ptr(), nat.stream(),
            ),
            "csb_attn_fwd_dense",
        )
        return out, lse
    qb, kb, qp, kp = _mask_ptrs(mask, B)
    nat.check(
        nat.lib().csb_attn_fwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B, Sq, Sk, Hq, Hk, D,
            q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0), out.stride(1), out.stride(0),
            scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp), cls.data_ptr(), st.data_ptr(),
            nat.stream(),
        ),
        "csb_attn_fwd",
    )
    return out, lse


def attention_backward(do, q, k, v, out, lse, mask: AttnMask, scale: float | None = None, dq=None, dk=None, dv=None):
    """Native backward; returns ``(dq, dk, dv)`` shaped like q, k, v."""
    B, Sq, Hq, D = q.shape
    Sk, Hk = k.shape[1], k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if do.stride(3) != 1 or do.stride(2) != D or do.stride(1) % 8:
        do = do.contiguous()
    dq = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty((B, Sk, Hk, D), dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty((B, Sk, Hk, D), dtype=q.dtype, device=q.device) if dv is None else dv
    dq_acc = torch.zeros((B, Sq, Hq, D), dtype=torch.float32, device=q.device)
    delta = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    cls = mask.classes(B, Sq, Sk, q.device)
    st = nat.status_word(q.device)
    ex, keep = mask.extras(B, Hq, Sq, Sk, q.device)
    if ex is not None:
        nat.check(
            nat.lib().csb_attn_bwd_dense(
                q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Sq, Sk, Hq, Hk, D,
                q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0), out.stride(1), out.stride(0),
                do.stride(1), do.stride(0), dq.stride(1), dq.stride(0), dk.stride(1), dk.stride(0), dv.stride(1),
                dv.stride(0), scale, mask.mode, cls.data_ptr(), C.addressof(ex), st.data_ptr(), nat.stream(),
            ),
            "csb_attn_bwd_dense",
        )
        return dq, dk, dv
    qb, kb, qp, kp = _mask_ptrs(mask, B)
    nat.check(
        nat.lib().csb_attn_bwd(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
            dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Sq, Sk, Hq, Hk, D,
            q.stride(1), q.stride(0), k.stride(1), k.stride(0), v.stride(1), v.stride(0), out.stride(1), out.stride(0),
            do.stride(1), do.stride(0), dq.stride(1), dq.stride(0), dk.stride(1), dk.stride(0), dv.stride(1),
            dv.stride(0), scale, mask.mode, nat.ptr(qb), nat.ptr(kb), nat.ptr(qp), nat.ptr(kp), cls.data_ptr(),
            st.data_ptr(), nat.stream(),
        ),
        "csb_attn_bwd",
    )
    return dq, dk, dv


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, scale):
        out, lse = attention_forward(q, k, v, mask, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mask, ctx.scale = mask, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(do, q, k, v, out, lse, ctx.mask, ctx.scale)
        return dq, dk, dv, None, None


class _AttnReplayFn(torch.autograd.Function):
    """Forward = an output computed earlier (kept across an activation recomputation); backward = the real one."""

    @staticmethod
    def forward(ctx, q, k, v, mask, scale, out, lse):
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mask, ctx.scale = mask, scale
        return out.view_as(out)

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = attention_backward(do, q, k, v, out, lse, ctx.mask, ctx.scale)
        return dq, dk, dv, None, None, None, None


_TAPE = threading.local()


class attention_tape:
    """Context manager used by activation recomputation that keeps attention outputs.

    ``record``: every :func:`attention` call appends its ``(out, lse)`` to ``items`` (the caller runs under
    ``torch.no_grad``).  ``replay``: calls pop their entry in the same order and skip the forward kernel; the
    backward kernel runs as usual.  ``out`` + ``lse`` cost ``S * H * (2 D + 4)`` bytes per layer, far less than the
    layer's other activations, while the forward kernel is the most expensive part of a recomputation at long
    sequence lengths.
    """

    def __init__(self, items: list, mode: str):
        assert mode in ("record", "replay")
        self.items, self.mode = items, mode

    def __enter__(self):
        self.prev = getattr(_TAPE, "cur", None)
        _TAPE.cur = self
        return self

    def __exit__(self, *exc):
        _TAPE.cur = self.prev
        return False


def attention_library(q, k, v, mask: AttnMask, scale=None) -> torch.Tensor:
    """PyTorch scaled-dot-product attention (flash / cuDNN / memory-efficient kernels): the library baseline.  Causal and
    full masks without explicit positions use the fused flags; everything else gets a dense boolean mask."""
    B, Sq = q.shape[:2]
    Sk = k.shape[1]
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    gqa = q.shape[2] != k.shape[2]
    plain = mask.q_pos is None and mask.k_pos is None
    if mask.bias is not None or mask.mode == MASK_DENSE:
        am = mask.bias.to(q.dtype) if mask.bias is not None else None
        if mask.mode == MASK_DENSE:
            keep = dense_mask(mask, B, Sq, Sk, q.device)[:, None]
            am = keep if am is None else am.masked_fill(~keep, float("-inf"))
        o = torch.nan_to_num(F.scaled_dot_product_attention(qh, kh, vh, attn_mask=am, scale=scale, enable_gqa=gqa))
        return o.transpose(1, 2)
    if mask.mode == MASK_CAUSAL and plain and Sq == Sk:
        o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale, enable_gqa=gqa)
    elif mask.mode == MASK_FULL:
        o = F.scaled_dot_product_attention(qh, kh, vh, scale=scale, enable_gqa=gqa)
    else:
        cache = mask._cls.get(("dense", B, Sq, Sk))
        if cache is None:
            cache = dense_mask(mask, B, Sq, Sk, q.device)[:, None]
            mask._cls[("dense", B, Sq, Sk)] = cache
        o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=cache, scale=scale, enable_gqa=gqa)
        o = torch.nan_to_num(o)  # fully masked (padding) rows
    return o.transpose(1, 2)


def attention(q, k, v, mask: AttnMask | None = None, scale: float | None = None) -> torch.Tensor:
    """``softmax(scale q k^T + mask) v`` for ``[B, S, H, D]`` tensors (GQA when ``Hq > Hk``)."""
    mask = mask or AttnMask.causal()
    if nat.LIBRARY_MODE and q.is_cuda:
        return attention_library(q, k, v, mask, scale)
    if q.is_cuda and q.dtype == torch.bfloat16:
        tape = getattr(_TAPE, "cur", None)
        if tape is not None and tape.mode == "record" and not torch.is_grad_enabled():
            out, lse = attention_forward(q, k, v, mask, scale)
            tape.items.append((out, lse))
            return out
        if tape is not None and tape.mode == "replay" and tape.items:
            out, lse = tape.items.pop(0)
            return _AttnReplayFn.apply(q, k, v, mask, scale, out, lse)
        return _AttnFn.apply(q, k, v, mask, scale)
    o, _ = attention_reference(q, k, v, mask, scale)
    return o
