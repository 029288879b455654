"""``bitfield_attn_func`` and ``BitfieldUtils``: the kernel-level API of the reference
(cornstarch/kernel/bitfield_attention.py:159-212,1269-1277) on the tcgen05 attention kernels."""

from __future__ import annotations

import torch

from ..ops import attention as A


def bitfield_attn_func(q, k, v, bitfield_mask, bias=None, softmax_scale=None, prefix_causal: bool = False):
    """``q``: ``[B, Sq, Hq, D]``; ``k, v``: ``[B, Sk, Hk, D]`` (GQA allowed); ``bitfield_mask``: int64 ``[B, S]``."""
    assert bias is None, "additive bias is not supported by the bitfield kernel"
    return A.attention(q, k, v, A.AttnMask.bitfield(bitfield_mask, prefix_causal=prefix_causal), softmax_scale)


class BitfieldUtils:
    """Cache of the per-step compressed (tile-class) mask, shared by all layers of a forward pass."""

    _cache: dict = {}

    @staticmethod
    def materialize_compressed_mask_from_bitfield_mask(bitfield_mask: torch.Tensor, block_m: int = 128,
                                                       block_n: int = 32) -> torch.Tensor:
        """int8 ``[B, ceil(S/block_m), ceil(S/block_n)]``: 0 = empty tile, 1 = partial, 2 = full."""
        key = (bitfield_mask.data_ptr(), tuple(bitfield_mask.shape), block_m, block_n, str(bitfield_mask.device))
        hit = BitfieldUtils._cache.get(key)
        if hit is not None:
            return hit
        B, S = bitfield_mask.shape
        cls = A.classify_mask(A.AttnMask.bitfield(bitfield_mask), B, S, S, bitfield_mask.device, block_m, block_n)
        BitfieldUtils._cache[key] = cls
        return cls

    @staticmethod
    def clear_cache():
        BitfieldUtils._cache.clear()
