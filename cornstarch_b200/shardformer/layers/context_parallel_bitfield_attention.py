"""Context-parallel bitfield attention at the reference's import path
(cornstarch/shardformer/layers/context_parallel_bitfield_attention.py:334-372).

The reference gathers K / V per head group with NCCL and runs a Triton kernel on the gathered tensors; here the local
queries attend keys and values that the kernel pulls from the owning GPUs (or, on other back ends, that one uneven
all-gather brings in), see :mod:`cornstarch_b200.parallel.cp`.
"""

from __future__ import annotations

import torch

from ...ops import attention as A
from ...parallel.cp import ContextParallelState, context_parallel_attention


def context_parallel_bitfield_attention_forward(module, query, key, value, bitfield_mask, compressed_mask=None,
                                                offsets_per_rank=None, sp_group=None, heads_stride: int = 1, dropout: float = 0.0,
                                                scaling=None, sliding_window=None, softcap=None, **kwargs):
    """``query / key / value``: ``[B, heads, S_local, D]`` (the layout attention interfaces of the reference receive);
    ``bitfield_mask``: int64 ``[B, S_total]`` over the WHOLE sequence; ``offsets_per_rank``: the token indices every rank
    holds.  ``compressed_mask``, ``heads_stride``, ``sliding_window`` and ``softcap`` are accepted for signature
    compatibility (tile classes are derived from the bitfields; the last two are ignored by the reference as well).
    Returns ``(output [B, S_local, heads, D], None)``."""
    assert bitfield_mask is not None and bitfield_mask.dtype == torch.int64, "bitfield attention needs an int64 attention mask"
    assert offsets_per_rank is not None and sp_group is not None
    assert not dropout, "attention dropout is not supported"
    state = ContextParallelState(sp_group, list(offsets_per_rank), A.AttnMask.bitfield(bitfield_mask), query.device)
    q, k, v = (t.transpose(1, 2).contiguous() for t in (query, key, value))
    return context_parallel_attention(q, k, v, state, scaling), None
