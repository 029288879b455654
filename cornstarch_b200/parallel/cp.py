"""Context parallelism: token -> rank assignment and attention over a sequence sharded across ranks.

Token assignment (``ContextParallelBatchSplitUtils``) reproduces the three modes of the reference
(cornstarch/shardformer/layers/utils.py:16-382): ``uniform`` (contiguous equal chunks), ``zigzag``
(2*sp chunks, rank i owns chunk i and chunk -i-1) and ``makespan_min`` (greedy longest-processing-time
over 128-token query blocks, the workload of a block being its number of non-empty 128x32 mask tiles
summed over the batch; ties resolved by a stable descending sort and a (load, rank) heap).  No split
happens when ``sp_size == 1`` or the sequence is shorter than ``128 * sp_size``.  Ranks may own
non-contiguous and unequal token sets; RoPE and the mask always use global token positions.

The per-block workload comes from the mask-classification kernel on the GPU (only ``B x S/128``
integers travel to the host), where the reference copies the whole compressed mask to the CPU every
step (utils.py:161-163).

Attention: K and V of all ranks are gathered (one stacked all-gather), the local queries attend to them
with the bitfield mask expressed through explicit positions, and dK/dV are reduce-scattered back — the
data flow of the reference's ``ContextParallelBitfieldAttention`` /``ContextParallelFlashAttention``
(cornstarch/shardformer/layers/context_parallel_bitfield_attention.py:17-331,
layers/context_parallel_attention.py) without its per-head loop.
"""

from __future__ import annotations

import heapq

import numpy as np
import torch
import torch.distributed as dist

from ..ops import attention as A
from ..shardformer.shard.shard_config import ContextParallelDistributionMode
from . import comm

BLOCK_M = 128
BLOCK_N = 32


class ContextParallelBatchSplitUtils:
    """Process-global cache of ``offsets_per_rank`` (list of int64 index tensors, one per sp rank)."""

    _offsets: list[torch.Tensor] | None = None

    @classmethod
    def set_context_parallel_offsets_cache(cls, offsets):
        cls._offsets = [torch.as_tensor(o, dtype=torch.long) for o in offsets] if offsets is not None else None

    @classmethod
    def get_context_parallel_offsets_cache(cls):
        return cls._offsets

    @classmethod
    def clear_cache(cls):
        cls._offsets = None

    # ------------------------------------------------------------------ partitioners (pure functions)
    @staticmethod
    def uniform(seq_len: int, sp_size: int) -> list[np.ndarray]:
        return [np.asarray(c) for c in np.array_split(np.arange(seq_len), sp_size)]

    @staticmethod
    def zigzag(seq_len: int, sp_size: int) -> list[np.ndarray]:
        chunks = np.array_split(np.arange(seq_len), 2 * sp_size)
        return [np.concatenate([chunks[i], chunks[-i - 1]]) for i in range(sp_size)]

    @staticmethod
    def block_workloads(mask: A.AttnMask | torch.Tensor, batch: int, seq_len: int, device) -> np.ndarray:
        """Per 128-row block: number of non-empty 128x32 tiles, summed over the batch."""
        if not isinstance(mask, A.AttnMask):
            mask = A.AttnMask.bitfield(mask)
        _cls, work = A.classify_mask(mask, batch, seq_len, seq_len, device, BLOCK_M, BLOCK_N, with_work=True)
        return work.sum(dim=0).cpu().numpy().astype(np.int64)

    @staticmethod
    def makespan_min(workloads: np.ndarray, seq_len: int, sp_size: int) -> list[np.ndarray]:
        order = np.argsort(-workloads, kind="stable")
        heap = [(0, r) for r in range(sp_size)]
        heapq.heapify(heap)
        assigned: list[list[int]] = [[] for _ in range(sp_size)]
        for blk in order:
            load, r = heapq.heappop(heap)
            heapq.heappush(heap, (load + int(workloads[blk]), r))
            assigned[r].append(int(blk))
        out = []
        for blocks in assigned:
            b = np.sort(np.asarray(blocks, dtype=np.int64))
            offs = (b[:, None] * BLOCK_M + np.arange(BLOCK_M)).ravel() if len(b) else np.zeros(0, dtype=np.int64)
            out.append(offs[offs < seq_len])
        return out

    # ------------------------------------------------------------------ dispatch
    @classmethod
    def create_context_parallel_split(cls, attention_mask, sp_group, dist_mode: ContextParallelDistributionMode | str,
                                      seq_len: int | None = None, batch: int | None = None, device=None):
        """Compute, cache and return ``offsets_per_rank``; ``None`` when no split applies."""
        sp_size = comm._world(sp_group)
        if isinstance(dist_mode, str):
            dist_mode = ContextParallelDistributionMode(dist_mode)
        bits = None
        if isinstance(attention_mask, A.AttnMask):
            bits = attention_mask.q_bits
        elif isinstance(attention_mask, torch.Tensor):
            bits = attention_mask
        if bits is not None:
            batch, seq_len = bits.shape
            device = bits.device
        if sp_size == 1 or seq_len is None or seq_len < BLOCK_M * sp_size:
            cls.set_context_parallel_offsets_cache(None)
            return None
        if dist_mode == ContextParallelDistributionMode.UNIFORM or (bits is None and dist_mode == ContextParallelDistributionMode.MAKESPAN_MIN):
            offs = cls.uniform(seq_len, sp_size)
        elif dist_mode == ContextParallelDistributionMode.ZIGZAG:
            offs = cls.zigzag(seq_len, sp_size)
        else:
            mask = attention_mask if isinstance(attention_mask, A.AttnMask) else A.AttnMask.bitfield(bits)
            full = A.AttnMask(mode=mask.mode, q_bits=mask.q_bits, k_bits=mask.k_bits)
            offs = cls.makespan_min(cls.block_workloads(full, batch, seq_len, device), seq_len, sp_size)
        cls.set_context_parallel_offsets_cache(offs)
        return cls._offsets

    @classmethod
    def split_batch(cls, batch: torch.Tensor, sp_group, dim: int = 1, is_label: bool = False) -> torch.Tensor:
        """Rows of ``dim`` owned by this rank (labels are shifted first so that position t predicts token t+1)."""
        if cls._offsets is None:
            return batch
        mine = cls._offsets[dist.get_rank(sp_group)].to(batch.device)
        if is_label:
            shifted = torch.full_like(batch, -100)
            shifted[:, :-1] = batch[:, 1:]
            batch = shifted
        return batch.index_select(dim, mine)

    @classmethod
    def get_local_compressed_mask(cls, compressed: torch.Tensor, sp_group) -> torch.Tensor:
        """Rows of my query blocks, columns reordered to the gathered-KV order (blocks of 128 rows / 32 columns)."""
        assert cls._offsets is not None
        rank = dist.get_rank(sp_group)
        qb = torch.unique(cls._offsets[rank] // BLOCK_M)
        kb = torch.unique_consecutive(torch.cat(cls._offsets) // BLOCK_N)
        return compressed[:, qb.to(compressed.device)][:, :, kb.to(compressed.device)]


class ContextParallelState:
    """What one forward pass needs: the sp group, offsets, and the mask seen by the local queries.

    The state rides on the :class:`AttnMask` handed to the layers (``mask._cp_state``), so an activation
    recomputation in the backward pass sees the state of its own micro-batch.
    """

    def __init__(self, group, offsets: list[torch.Tensor] | None, full_mask: A.AttnMask | None, device):
        self.group = group
        self.rank = dist.get_rank(group)
        if offsets is None:
            # encoders: contiguous uniform chunks, full attention; only the gather sizes are needed (exchanged lazily)
            self.sizes, self.mine, self.all = None, None, None
            self.local_mask = A.AttnMask.full()
        else:
            self.sizes = [int(o.numel()) for o in offsets]
            self.mine = offsets[self.rank].to(device)
            self.all = torch.cat(offsets).to(device)
            self.local_mask = self._localize(full_mask)
        self.local_mask._cp_state = self

    def _localize(self, m: A.AttnMask | None) -> A.AttnMask:
        if m is None:
            m = A.AttnMask.causal()
        B = m.q_bits.shape[0] if m.q_bits is not None else 1
        q_pos = self.mine.int()[None].expand(B, -1).contiguous()
        k_pos = self.all.int()[None].expand(B, -1).contiguous()
        qb = m.q_bits.index_select(1, self.mine) if m.q_bits is not None else None
        kb = (m.k_bits if m.k_bits is not None else m.q_bits)
        kb = kb.index_select(1, self.all) if kb is not None else None
        return A.AttnMask(mode=m.mode, q_bits=qb, k_bits=kb, q_pos=q_pos, k_pos=k_pos)


FUSED_CP_ENABLED = True  # stream K/V tiles from the peers inside the attention kernels instead of gathering with NCCL


def _fused_for(state: "ContextParallelState", q):
    from ..ops import _native as nat

    if nat.LIBRARY_MODE or not FUSED_CP_ENABLED or state.sizes is None or not q.is_cuda or q.dtype != torch.bfloat16:
        return None
    from .cp_fused import FusedContextParallelAttention

    return FusedContextParallelAttention.get(state.group)


def context_parallel_attention(q, k, v, state: ContextParallelState, scale=None, mask: A.AttnMask | None = None):
    """Local queries against the gathered keys/values (``[B, S_local, H, D]`` in, same out)."""
    fused = _fused_for(state, q)
    if fused is not None:
        from .cp_fused import fused_context_parallel_attention, padded_mask

        if getattr(state, "fused_mask", None) is None:
            state.fused_mask = padded_mask(mask or state.local_mask, state.sizes)
        return fused_context_parallel_attention(q, k, v, fused, state.sizes, state.fused_mask, scale)
    kv = torch.stack([k, v], dim=0)  # one collective for both
    kv_all = comm.gather_forward_reduce_scatter_backward(kv, 2, state.group, state.sizes)
    return A.attention(q, kv_all[0], kv_all[1], mask or state.local_mask, scale)


def _cp_attn_impl(q, k, v, mask, scale):
    st = getattr(mask, "_cp_state", None)
    if st is None:
        return A.attention(q, k, v, mask, scale)
    return context_parallel_attention(q, k, v, st, scale, mask)


def install_context_parallel_attention(model, sp_group) -> None:
    """Route every attention module of ``model`` through :func:`context_parallel_attention`.

    The model's forward attaches the per-step :class:`ContextParallelState` to the mask it hands to its layers.
    """
    for mod in model.modules():
        if hasattr(mod, "attn_impl"):
            mod.attn_impl = _cp_attn_impl
    model._cp_group = sp_group
