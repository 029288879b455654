"""Context-parallel full attention for encoders at the reference's import path
(cornstarch/shardformer/layers/context_parallel_attention.py:17-283: per-head all-gather of K / V and FlashAttention-2 on
the gathered tensors).  Here: one uneven exchange (or the peer-memory path) and this package's attention kernel."""

from __future__ import annotations

from ...parallel.cp import ContextParallelState, context_parallel_attention


def context_parallel_flash_attention_forward(module, query, key, value, attention_mask=None, sp_group=None, dropout: float = 0.0,
                                             scaling=None, **kwargs):
    """``query / key / value``: ``[B, heads, S_local, D]``; full (bidirectional) attention over the tokens of all ranks of
    ``sp_group``; shards may have different lengths.  Returns ``(output [B, S_local, heads, D], None)``."""
    assert sp_group is not None and not dropout
    state = ContextParallelState(sp_group, None, None, query.device)
    q, k, v = (t.transpose(1, 2).contiguous() for t in (query, key, value))
    return context_parallel_attention(q, k, v, state, scaling), None
