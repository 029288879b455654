"""Expert parallelism: every rank of an expert-parallel group owns ``num_experts / ep`` experts; tokens travel
to the owners of their top-k experts (dispatch), run through the expert MLPs there, and travel back (combine).

The reference has no expert parallelism (its Mixtral / Qwen3-MoE experts are tensor-parallel only,
cornstarch/shardformer/policies/mixtral.py:216-234, and every rank loops over all experts,
cornstarch/shardformer/modeling/mixtral.py); this is the capability its MoE configuration needs on a
multi-GPU node.

Data movement per MoE layer::

    sort (token, k) pairs by expert            -> rows grouped by destination rank
    counts[ep, local] --all-to-all-->           recv_counts[src, local]
    rows   --uneven all-to-all-->               rows grouped by (src, local expert)
    regroup by local expert, one SwiGLU per contiguous segment (three tcgen05 GEMMs each)
    results --uneven all-to-all back-->         rows in the sender's sorted order
    scale by routing weight, index_add into the token order

Both all-to-alls are autograd functions whose backward is the reverse exchange.  On NCCL they are
``all_to_all_single`` with split sizes; on gloo (CPU tests) they are emulated with a padded all-gather.

Capacity mode (``ExpertParallel(..., capacity_factor=f)`` / ``shard_experts(..., capacity_factor=f)``) is the same layer
with STATIC shapes: every rank sends exactly ``C = ceil(f * tokens * k / num_experts)`` rows per expert (unused slots are
zero rows, pairs beyond an expert's capacity are dropped and counted in ``dropped_pairs``), so both exchanges are
all-to-alls with equal splits and nothing is read back to the host: no count exchange, no synchronisation, every tensor
shape fixed from step to step.  ``tokens`` is the token count of the call, which must then be equal on all ranks, or the
fixed ``capacity_tokens`` (an upper bound) when ranks see batches of different lengths.  The price is the padding (``f - 1`` of the expert GEMM rows at balanced load) and, like the
capacity factor of GShard / Switch layers, dropped pairs when one expert receives more than ``f`` times its share.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a_uneven(x: torch.Tensor, send: list[int], recv: list[int], group) -> torch.Tensor:
    out = x.new_empty((sum(recv), *x.shape[1:]))
    if dist.get_backend(group) != "gloo":
        dist.all_to_all_single(out, x.contiguous(), recv, send, group=group)
        return out
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    mx = torch.tensor([max(send) if send else 0], dtype=torch.int64)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    mx = int(mx.item())
    buf = x.new_zeros((ws, mx, *x.shape[1:]))
    start = 0
    for d, n in enumerate(send):
        buf[d, :n] = x[start : start + n]
        start += n
    everyone = [torch.empty_like(buf) for _ in range(ws)]
    dist.all_gather(everyone, buf, group=group)
    start = 0
    for s, n in enumerate(recv):
        out[start : start + n] = everyone[s][rank, :n]
        start += n
    return out


class _AllToAllUneven(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        return _a2a_uneven(x, send, recv, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_uneven(g.contiguous(), ctx.recv, ctx.send, ctx.group), None, None, None


def all_to_all_uneven(x, send_splits: list[int], recv_splits: list[int], group):
    return _AllToAllUneven.apply(x, send_splits, recv_splits, group)


def expert_counts(flat_e: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Pairs per expert.  Not ``torch.bincount``: on a device that reads the smallest and largest value on the host."""
    return torch.zeros(num_experts, dtype=torch.long, device=flat_e.device).scatter_add_(0, flat_e, torch.ones_like(flat_e))


def by_expert_order(recv_counts: torch.Tensor, total: int) -> torch.Tensor:
    """Permutation that takes received rows from (source rank, local expert) order to (local expert, source rank) order.
    ``recv_counts[src, local]`` stays on its device; ``total`` (their sum, known on the host) sizes the result, so nothing
    is read back and nothing is copied in."""
    ws, local = recv_counts.shape
    expert_of_segment = torch.arange(local, device=recv_counts.device).repeat(ws)
    keys = torch.repeat_interleave(expert_of_segment, recv_counts.reshape(-1), output_size=total)
    return torch.argsort(keys, stable=True)


FUSED_EP_ENABLED = True  # exchange tokens with this package's peer-memory kernel instead of NCCL all_to_all


ONE_PROCESS = "one process"  # in place of a process group: every expert is local and nothing is exchanged


class ExpertParallel:
    """Attached to a sparse MoE block as ``block.ep``; the block then holds only this rank's experts."""

    def __init__(self, group, num_experts: int, capacity_factor: float | None = None, capacity_tokens: int | None = None):
        self.capacity_factor = capacity_factor
        # capacity mode sizes its exchange from the number of tokens of a call, which must then be the same on every rank.
        # With capacity_tokens the size comes from this fixed number instead (an upper bound of the tokens per call and
        # rank): batches of different lengths on different ranks still exchange buffers of one static shape.
        self.capacity_tokens = capacity_tokens
        self.dropped_pairs = None  # capacity mode: device scalar, pairs dropped in the last call (read it when convenient)
        self.group = group
        # ONE_PROCESS: no process group at all (capacity mode of a single process: static shapes and the grouped GEMM
        # without any exchange)
        self.ws = 1 if group is ONE_PROCESS else dist.get_world_size(group)
        self.rank = 0 if group is ONE_PROCESS else dist.get_rank(group)
        assert group is not ONE_PROCESS or capacity_factor is not None, "a single process without a group runs the capacity form"
        assert num_experts % self.ws == 0, f"{num_experts} experts cannot be split over {self.ws} ranks"
        self.num_experts = num_experts
        self.local = num_experts // self.ws
        self.first = self.rank * self.local
        self.last_recv_tokens = 0  # tokens this rank's experts processed in the last call (load statistics)

    def local_expert_ids(self) -> range:
        return range(self.first, self.first + self.local)

    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``counts[E]`` rows I send per expert -> ``recv[src, local]`` rows I receive per source and local expert."""
        send = counts.view(self.ws, self.local).contiguous()
        if dist.get_backend(self.group) == "gloo":
            everyone = [torch.empty_like(send) for _ in range(self.ws)]
            dist.all_gather(everyone, send, group=self.group)
            return torch.stack([e[self.rank] for e in everyone], dim=0)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        return recv

    def forward(self, x2: torch.Tensor, weights: torch.Tensor, experts_idx: torch.Tensor, experts, act: str) -> torch.Tensor:
        T, H = x2.shape
        k = experts_idx.shape[1]
        if self.capacity_factor is not None:
            return self._forward_capacity(x2, weights, experts_idx, experts, act)
        flat_e = experts_idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        token_of = torch.div(order, k, rounding_mode="floor")
        counts = expert_counts(flat_e, self.num_experts)
        fused = self._fused(x2)
        if fused is not None:
            return self._forward_fused(fused, x2, weights, order, token_of, counts, experts, act)
        rec = _replayed_counts()
        if rec is None:
            recv_counts = self.exchange_counts(counts)
            # one host read for both directions' split sizes: the only point of this path where the host waits
            rec = (torch.cat([counts.view(self.ws, self.local).sum(1), recv_counts.reshape(-1)]).tolist(), recv_counts)
            _record_counts(rec)
        both, recv_counts = rec
        send_splits = both[: self.ws]
        rc = [both[self.ws + s * self.local : self.ws + (s + 1) * self.local] for s in range(self.ws)]
        recv_splits = [sum(r) for r in rc]
        rows = all_to_all_uneven(x2[token_of], send_splits, recv_splits, self.group)  # grouped by (src, local expert)
        self.last_recv_tokens = rows.shape[0]
        if self.local > 1:
            perm = by_expert_order(recv_counts, rows.shape[0])
            rows = rows[perm]
        outs, start = [], 0
        for e in range(self.local):
            n = sum(rc[s][e] for s in range(self.ws))
            seg = rows[start : start + n]
            # an expert that received nothing still takes part in autograd (its weights get zero gradients)
            outs.append(experts[e](seg, act))
            start += n
        y = torch.cat(outs, dim=0) if len(outs) > 1 else outs[0]
        if self.local > 1:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel(), device=perm.device)
            y = y[inv]
        back = all_to_all_uneven(y, recv_splits, send_splits, self.group)
        back = back * weights.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
        out = torch.zeros_like(x2)
        out.index_add_(0, token_of, back)
        return out

    def _forward_capacity(self, x2, weights, experts_idx, experts, act):
        """Static-shape dispatch / combine (see the module docstring): no host reads, equal-split all-to-alls."""
        import math

        T, H = x2.shape
        k = experts_idx.shape[1]
        E, ws, L = self.num_experts, self.ws, self.local
        C = max(1, math.ceil(self.capacity_factor * (self.capacity_tokens or T) * k / E))
        if x2.is_cuda:
            # every expert then holds a multiple of 256 rows: whole tiles of the grouped GEMM that runs all local experts
            step = 256 // math.gcd(256, ws)
            C = (C + step - 1) // step * step
        flat_e = experts_idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        sorted_e = flat_e[order]
        token_of = torch.div(order, k, rounding_mode="floor")
        counts = expert_counts(flat_e, E)
        starts = torch.cumsum(counts, 0) - counts
        pos = torch.arange(T * k, device=x2.device) - starts[sorted_e]  # rank of a pair among its expert's pairs
        keep = pos < C
        self.dropped_pairs = (~keep).sum()
        dump = E * C  # one extra row that collects every dropped pair
        slot = torch.where(keep, sorted_e * C + pos, torch.full_like(pos, dump))
        send = x2.new_zeros((E * C + 1, H)).index_copy(0, slot, x2[token_of])[:dump]
        recv = _AllToAllEqual.apply(send.view(ws, L * C, H), self.group)  # [src, (local expert, slot), H]
        self.last_recv_tokens = ws * L * C
        per_expert = recv.view(ws, L, C, H).transpose(0, 1).reshape(L, ws * C, H)
        from ..models.moe import experts_forward_grouped

        y = experts_forward_grouped(experts, per_expert, act)  # zero rows stay zero through a bias-free gated MLP
        y = y.view(L, ws, C, H).transpose(0, 1).reshape(ws, L * C, H)
        back = _AllToAllEqual.apply(y, self.group).reshape(dump, H)
        back = torch.cat([back, back.new_zeros((1, H))], dim=0)[slot]  # dropped pairs read the zero row
        back = back * weights.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
        out = torch.zeros_like(x2)
        out.index_add_(0, token_of, back)
        return out

    def _fused(self, x2):
        from ..ops import _native as nat

        if nat.LIBRARY_MODE or not FUSED_EP_ENABLED or not x2.is_cuda or x2.dtype != torch.bfloat16 or x2.shape[1] % 8:
            return None
        from .ep_fused import FusedExpertExchange

        return FusedExpertExchange.get(self.group)

    def _forward_fused(self, ex, x2, weights, order, token_of, counts, experts, act):
        """Same data flow as ``forward`` with both exchanges done by the peer-memory push kernel."""
        from .ep_fused import fused_all_to_all

        T, H = x2.shape
        k = order.numel() // T
        rec = _replayed_counts()
        if rec is None:
            everyone = [torch.empty_like(counts) for _ in range(self.ws)]
            dist.all_gather(everyone, counts, group=self.group)  # counts[src][expert]: placement of every rank's rows
            stacked = torch.stack(everyone).view(self.ws, self.ws, self.local)  # [src][dst][local expert]
            rec = (stacked.tolist(), stacked[:, self.rank].contiguous())
            _record_counts(rec)
        mat, recv_counts = rec
        send = [[sum(mat[s][d]) for d in range(self.ws)] for s in range(self.ws)]
        # every rank may receive at most all (token, k) pairs of the group; sized once from the first call's total
        total_pairs = sum(sum(r) for r in send)
        ex.ensure(max(ex.capacity_rows, total_pairs), H)
        rows = fused_all_to_all(x2, token_of, send, ex)  # gather by token fused into the push
        me = self.rank
        rc = [mat[s][me] for s in range(self.ws)]
        self.last_recv_tokens = rows.shape[0]
        perm = None
        if self.local > 1:
            perm = by_expert_order(recv_counts, rows.shape[0])
            rows = rows[perm]
        outs, start = [], 0
        for e in range(self.local):
            n = sum(rc[s][e] for s in range(self.ws))
            outs.append(experts[e](rows[start : start + n], act))
            start += n
        y = torch.cat(outs, dim=0) if len(outs) > 1 else outs[0]
        if perm is not None:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel(), device=perm.device)
            y = y[inv]
        rev = [[send[d][s] for d in range(self.ws)] for s in range(self.ws)]
        back = fused_all_to_all(y, None, rev, ex)
        back = back * weights.reshape(-1)[order].unsqueeze(-1).to(back.dtype)
        out = torch.zeros_like(x2)
        out.index_add_(0, token_of, back)
        return out


def _a2a_equal(x: torch.Tensor, group) -> torch.Tensor:
    """All-to-all with equal splits: ``x`` is ``[world, n, ...]``, slice ``d`` goes to rank ``d``."""
    if group is ONE_PROCESS:
        return x
    if dist.get_backend(group) != "gloo":
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=group)
        return out
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    everyone = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(everyone, x.contiguous(), group=group)
    return torch.stack([e[rank] for e in everyone], dim=0)


class _AllToAllEqual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_equal(x, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_equal(g.contiguous(), ctx.group), None


def _replayed_counts():
    """Inside the recomputation of a layer the routing is the one of the first forward pass: the token counts that pass
    exchanged (a collective plus a host read) are taken from the recomputation tape instead of being exchanged again."""
    from ..ops.attention import _TAPE

    tape = getattr(_TAPE, "cur", None)
    if tape is None or tape.mode != "replay":
        return None
    tag, value = tape.items.pop(0)
    assert tag == "ep_counts", "recomputation tape out of order"
    return value


def _record_counts(value) -> None:
    from ..ops.attention import _TAPE

    tape = getattr(_TAPE, "cur", None)
    if tape is not None and tape.mode == "record":
        tape.items.append(("ep_counts", value))


def shard_experts(model, group, capacity_factor: float | None = None,
                  capacity_tokens: int | None = None) -> list[torch.nn.Parameter]:
    """Keep only this rank's experts in every sparse MoE block of ``model`` and attach the exchange.

    Returns the expert parameters (they are NOT replicated over the group: no data-parallel reduction, and an
    optimizer must not shard them again)."""
    import torch.nn as nn

    expert_params = []
    for m in model.modules():
        if hasattr(m, "experts") and hasattr(m, "ep") and isinstance(m.experts, nn.ModuleList):
            if m.ep is not None:
                continue
            ep = ExpertParallel(group, len(m.experts), capacity_factor, capacity_tokens)
            m.experts = nn.ModuleList([m.experts[i] for i in ep.local_expert_ids()])
            m.ep = ep
            expert_params += list(m.experts.parameters())
            _install_global_expert_names(m, ep)
    for p in expert_params:
        p.expert_parallel = True
    return expert_params


def set_expert_capacity(model, capacity_factor: float) -> None:
    """Capacity mode for a model whose experts all live in this process (no expert parallelism, no process group): every
    sparse block routes with static shapes, reads nothing on the host and runs its experts through one grouped GEMM per
    projection.  Pairs beyond ``capacity_factor`` times an expert's fair share are dropped (``dropped_pairs``)."""
    import torch.nn as nn

    for m in model.modules():
        if hasattr(m, "experts") and hasattr(m, "ep") and isinstance(m.experts, nn.ModuleList):
            assert m.ep is None or m.ep.group is ONE_PROCESS, "this block's experts are already sharded over a group"
            m.ep = ExpertParallel(ONE_PROCESS, len(m.experts), capacity_factor)


def dropped_pairs(model) -> torch.Tensor | None:
    """Capacity mode: (token, expert) pairs that the last forward pass of ``model`` dropped on this rank, summed over its
    sparse blocks, as a device scalar (reading it is the caller's synchronisation).  ``None`` without capacity mode."""
    total = None
    for m in model.modules():
        ep = getattr(m, "ep", None)
        if isinstance(ep, ExpertParallel) and ep.dropped_pairs is not None:
            total = ep.dropped_pairs if total is None else total + ep.dropped_pairs
    return total


def _install_global_expert_names(block, ep: ExpertParallel) -> None:
    """Checkpoints name experts by their global index: ``experts.<local>`` <-> ``experts.<first + local>`` on save / load."""
    import re

    first, local = ep.first, ep.local

    def on_save(module, state_dict, prefix, local_metadata):
        pat = re.compile(re.escape(prefix) + r"experts\.(\d+)\.")
        for k in [k for k in state_dict if pat.match(k)]:
            j = int(pat.match(k).group(1))
            state_dict[pat.sub(f"{prefix}experts.{first + j}.", k, count=1)] = state_dict.pop(k)
        return state_dict

    def on_load(module, state_dict, prefix, *args):
        pat = re.compile(re.escape(prefix) + r"experts\.(\d+)\.")
        renamed = {}
        for k in [k for k in state_dict if pat.match(k)]:
            e = int(pat.match(k).group(1))
            v = state_dict.pop(k)
            if first <= e < first + local:
                renamed[pat.sub(f"{prefix}experts.{e - first}.", k, count=1)] = v
        state_dict.update(renamed)

    block._register_state_dict_hook(on_save)
    block.register_load_state_dict_pre_hook(on_load)


def gather_full_state_dict(model, group, dst: int = 0) -> dict | None:
    """The unsharded state dict (all experts, global names) on rank ``dst`` of the group, ``None`` elsewhere.
    Replicated parameters are taken from ``dst``; expert parameters travel as CPU tensors through the group."""
    import re

    sd = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    mine = {k: v for k, v in sd.items() if re.search(r"\.experts\.\d+\.", k)}
    everyone = [None] * dist.get_world_size(group)
    dist.all_gather_object(everyone, mine, group=group)
    if dist.get_rank(group) != dst:
        return None
    for part in everyone:
        sd.update(part)
    return dict(sorted(sd.items()))
