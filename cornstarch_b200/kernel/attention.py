"""``flash_attn_func`` with a dense boolean mask (the reference's cornstarch/kernel/attention.py:1126-1147), and the
packed variable-length entry points.

A dense ``[B, Sq, Sk]`` mask cannot be expressed as a bitfield in general: the kernels take it as a byte matrix
(mask mode ``MASK_DENSE``), classify its 128 x 128 tiles once and read it only inside tiles that mix allowed and
masked pairs; an additive bias is added to the scores in the kernel.  Multimodal training uses the bitfield path.
"""

from __future__ import annotations

import torch

from ..ops import attention as A


def flash_attn_func(q, k, v, bias=None, mask=None, softmax_scale=None):
    """``q, k, v``: ``[B, S, H, D]``; ``mask``: bool ``[B, Sq, Sk]`` (True = attend); ``bias`` broadcastable to ``[B, H, Sq, Sk]``
    (no gradient flows to it, as in the reference).  Runs on the attention kernels: the dense mask is read tile by tile
    (tiles without an allowed pair are skipped, tiles with every pair allowed skip the mask), the bias is added to the
    scores inside the kernel."""
    if mask is None and bias is None:
        return A.attention(q, k, v, A.AttnMask.full(), softmax_scale)
    return A.attention(q, k, v, A.AttnMask.from_dense(mask, bias), softmax_scale)


_MAX_PACKED_SEQUENCES = 60  # one mask bit per packed sequence; bit 0 is the text (causal) bit


def _sequence_ids(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    """``[total]`` index of the sequence every packed token belongs to."""
    return torch.bucketize(torch.arange(total, device=cu_seqlens.device), cu_seqlens[1:].long(), right=True)


def flash_attn_varlen_func(q, k, v, cu_seqlens, max_seqlen: int | None = None, dropout_p: float = 0.0,
                           softmax_scale=None, causal: bool = False):
    """Attention over sequences packed along the first dimension: ``q, k, v`` are ``[total, H, D]`` and sequence ``i``
    occupies rows ``cu_seqlens[i]:cu_seqlens[i + 1]`` (the calling convention of flash-attn's varlen functions, which
    the reference uses for InternViT, cornstarch/models/intern_vit/flash_attention.py:52-100).

    Up to 60 sequences run as ONE masked sequence on the bitfield kernel: a token carries the bit of its sequence, so the
    tile map skips every tile that pairs two sequences and nothing is padded.  More sequences are padded to
    ``[n, max_seqlen]`` with the padding masked out.  Dropout is not supported (``dropout_p`` must be 0)."""
    assert dropout_p == 0.0, "attention dropout is not supported"
    total, n = q.shape[0], cu_seqlens.numel() - 1
    if n <= _MAX_PACKED_SEQUENCES:
        bit = (torch.ones(total, dtype=torch.int64, device=q.device) << (1 + _sequence_ids(cu_seqlens, total)))[None]
        mask = A.AttnMask.bitfield(bit | 1, k_bits=bit) if causal else A.AttnMask.bitfield(bit)
        return A.attention(q[None], k[None], v[None], mask, softmax_scale)[0]
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    S = int(max_seqlen) if max_seqlen is not None else int(lens.max())
    seq = _sequence_ids(cu_seqlens, total)
    col = torch.arange(total, device=q.device) - cu_seqlens[:-1].long()[seq]
    text = (1 << 62) | 1

    def pad(t):
        out = t.new_zeros(n, S, *t.shape[1:])
        out[seq, col] = t
        return out

    bits = torch.zeros(n, S, dtype=torch.int64, device=q.device)
    bits[seq, col] = text if causal else 2
    o = A.attention(pad(q), pad(k), pad(v), A.AttnMask.bitfield(bits), softmax_scale)
    return o[seq, col]


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen: int | None = None, dropout_p: float = 0.0,
                                     softmax_scale=None, causal: bool = False):
    """``qkv``: ``[total, 3, H, D]``; see :func:`flash_attn_varlen_func`."""
    return flash_attn_varlen_func(qkv[:, 0], qkv[:, 1], qkv[:, 2], cu_seqlens, max_seqlen, dropout_p, softmax_scale, causal)


class FlashAttention(torch.nn.Module):
    """Module form with the call signature of the reference's InternViT attention core
    (cornstarch/models/intern_vit/flash_attention.py:14-110): ``qkv`` is ``[B, S, 3, H, D]`` with an optional boolean
    ``key_padding_mask [B, S]`` (True = real token), or ``[total, 3, H, D]`` with ``cu_seqlens``.  Returns
    ``(output, None)``; padded positions of the output are zero."""

    def __init__(self, softmax_scale=None, attention_dropout: float = 0.0, device=None, dtype=None):
        super().__init__()
        assert attention_dropout == 0.0, "attention dropout is not supported"
        self.softmax_scale = softmax_scale

    def forward(self, qkv, key_padding_mask=None, causal: bool = False, cu_seqlens=None, max_s=None, need_weights: bool = False):
        assert not need_weights
        if cu_seqlens is not None:
            return flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_s, 0.0, self.softmax_scale, causal), None
        q, k, v = qkv.unbind(dim=2)
        if key_padding_mask is None:
            mask = A.AttnMask.causal() if causal else A.AttnMask.full()
            return A.attention(q, k, v, mask, self.softmax_scale), None
        keep = key_padding_mask.bool()
        bits = torch.where(keep, torch.full_like(keep, (1 << 62) | 1 if causal else 2, dtype=torch.int64),
                           torch.zeros_like(keep, dtype=torch.int64))
        out = A.attention(q, k, v, A.AttnMask.bitfield(bits), self.softmax_scale)
        return out * keep[:, :, None, None].to(out.dtype), None
