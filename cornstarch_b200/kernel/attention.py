"""``flash_attn_func`` with a dense boolean mask (the reference's cornstarch/kernel/attention.py:1126-1147).

A dense ``[B, Sq, Sk]`` mask cannot be expressed as a bitfield in general, so this entry point runs the
math in PyTorch (fp32 softmax) when a mask is given; with ``mask=None`` it is full attention on the
tcgen05 kernel.  Multimodal training uses the bitfield path, which is the fused one.
"""

from __future__ import annotations

import math

import torch

from ..ops import attention as A


def flash_attn_func(q, k, v, bias=None, mask=None, softmax_scale=None):
    """``q, k, v``: ``[B, S, H, D]``; ``mask``: bool ``[B, Sq, Sk]`` (True = attend); ``bias`` broadcastable to ``[B, H, Sq, Sk]``."""
    if mask is None and bias is None:
        return A.attention(q, k, v, A.AttnMask.full(), softmax_scale)
    scale = softmax_scale or 1.0 / math.sqrt(q.shape[-1])
    g = q.shape[2] // k.shape[2]
    qf = q.permute(0, 2, 1, 3).float()
    kf = k.permute(0, 2, 1, 3).float().repeat_interleave(g, dim=1)
    vf = v.permute(0, 2, 1, 3).float().repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if bias is not None:
        s = s + bias.float()
    if mask is not None:
        m = mask[:, None].bool()
        s = s.masked_fill(~m, float("-inf"))
    lse = torch.logsumexp(s, dim=-1, keepdim=True)
    p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse))
    if mask is not None:
        p = torch.where(m, p, torch.zeros_like(p))
    return torch.matmul(p, vf).permute(0, 2, 1, 3).to(q.dtype)
