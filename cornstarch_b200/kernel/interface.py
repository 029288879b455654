"""Bitfield attention mask construction and the attention-interface adapters.

``create_bitfield_attention_mask`` encodes one int64 per token: text tokens carry bit 0, bit 62 and
every modality bit (so text attends causally to text and to every modality); tokens of modality ``i``
carry only bit ``i + 1`` (bidirectional attention inside the modality); 0 marks padding.  This is the
builder whose output the reference kernel tests use (cornstarch/kernel/interface.py:13-30,
tests/test_kernel/test_bitfield_attention.py:164 in the reference).

``create_instance_bitfield_attention_mask`` gives every modality *instance* (e.g. each image of an
interleaved sample) its own bit, to be used with ``prefix_causal=True``: an image then attends
bidirectionally to itself and causally to everything before it.
"""

from __future__ import annotations

import torch

from ..ops import attention as A

TEXT_BITS = (1 << 62) | 1
MAX_MODALITY_BITS = 61


def _native_mask(input_ids: torch.Tensor, ids: list[int], padding_mask, instance: bool) -> torch.Tensor | None:
    """The mask built by one launch of ``csb_bitfield_mask`` for int64 CUDA ids; ``None`` = use the PyTorch statement."""
    import ctypes as C

    from ..ops import _native as nat

    if not (input_ids.is_cuda and input_ids.dtype == torch.int64 and input_ids.dim() == 2) or nat.LIBRARY_MODE:
        return None
    nat.declare("csb_bitfield_mask", [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p])
    x = input_ids.contiguous()
    pad = None
    if padding_mask is not None:
        pad = padding_mask.to(device=x.device).ne(0).to(torch.uint8).contiguous()
    out = torch.empty_like(x)
    arr = (C.c_long * max(1, len(ids)))(*[int(i) for i in ids])
    nat.check(nat.lib().csb_bitfield_mask(x.data_ptr(), C.cast(arr, C.c_void_p), len(ids), nat.ptr(pad), out.data_ptr(),
                                          x.shape[0], x.shape[1], int(instance), nat.stream()), "csb_bitfield_mask")
    return out


def create_bitfield_attention_mask(input_ids: torch.Tensor, token_ids: dict[str, int] | list[int],
                                   padding_mask: torch.Tensor | None = None) -> torch.Tensor:
    """int64 ``[B, S]`` bitfield mask from placeholder token ids (dict order = bit order)."""
    ids = list(token_ids.values()) if isinstance(token_ids, dict) else list(token_ids)
    assert len(ids) <= MAX_MODALITY_BITS, "at most 61 modalities fit the bitfield"
    native = _native_mask(input_ids, ids, padding_mask, instance=False)
    if native is not None:
        return native
    text = TEXT_BITS
    for i in range(len(ids)):
        text |= 1 << (i + 1)
    mask = torch.full_like(input_ids, text, dtype=torch.int64)
    for i, tid in enumerate(ids):
        mask = torch.where(input_ids == tid, torch.full_like(mask, 1 << (i + 1)), mask)
    if padding_mask is not None:
        mask = torch.where(padding_mask.bool(), mask, torch.zeros_like(mask))
    return mask


def create_instance_bitfield_attention_mask(input_ids: torch.Tensor, token_ids: dict[str, int] | list[int],
                                            padding_mask: torch.Tensor | None = None) -> torch.Tensor:
    """One bit per contiguous run of modality placeholder tokens (bits are reused modulo 61)."""
    ids = list(token_ids.values()) if isinstance(token_ids, dict) else list(token_ids)
    native = _native_mask(input_ids, ids, padding_mask, instance=True) if len(ids) <= MAX_MODALITY_BITS else None
    if native is not None:
        return native
    is_modal = torch.zeros_like(input_ids, dtype=torch.bool)
    for tid in ids:
        is_modal |= input_ids == tid
    prev = torch.zeros_like(input_ids)
    prev[:, 1:] = input_ids[:, :-1]
    prev_modal = torch.zeros_like(is_modal)
    prev_modal[:, 1:] = is_modal[:, :-1]
    starts = is_modal & (~prev_modal | (prev != input_ids))
    inst = torch.cumsum(starts.long(), dim=1) - 1  # instance number of each modality token
    bit = (inst % MAX_MODALITY_BITS) + 1
    text = TEXT_BITS | (((1 << MAX_MODALITY_BITS) - 1) << 1)
    mask = torch.where(is_modal, torch.ones_like(input_ids, dtype=torch.int64) << bit, torch.full_like(input_ids, text, dtype=torch.int64))
    if padding_mask is not None:
        mask = torch.where(padding_mask.bool(), mask, torch.zeros_like(mask))
    return mask


def bitfield_attention_forward(module, query, key, value, attention_mask, scaling=None, dropout=0.0, sliding_window=None,
                               softcap=None, **kwargs):
    """HF attention-interface signature: ``[B, H, S, D]`` inputs, int64 ``[B, S]`` bitfield mask.

    ``sliding_window`` and ``softcap`` are accepted and ignored, as in the reference adapter
    (cornstarch/kernel/interface.py:56-67).  Returns ``([B, S, H, D], None)``.
    """
    q, k, v = (t.transpose(1, 2) for t in (query, key, value))
    if not (q.stride(3) == 1 and q.stride(2) == q.shape[3]):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    mask = attention_mask if isinstance(attention_mask, A.AttnMask) else A.AttnMask.bitfield(attention_mask)
    return A.attention(q, k, v, mask, scaling), None


def cornstarch_attention_forward(module, query, key, value, attention_mask, scaling=None, dropout=0.0, **kwargs):
    """Same adapter for a dense boolean mask ``[B, Sq, Sk]`` (or ``None`` = full attention)."""
    q, k, v = (t.transpose(1, 2).contiguous() for t in (query, key, value))
    if attention_mask is None:
        return A.attention(q, k, v, A.AttnMask.full(), scaling), None
    from .attention import flash_attn_func

    return flash_attn_func(q, k, v, mask=attention_mask, softmax_scale=scaling), None
