"""Differentiable collectives used by the tensor / sequence / context parallel layers.

These are the autograd-aware wrappers the reference gets from ColossalAI
(``gather_forward_split_backward``, ``split_forward_gather_backward``, ``all_to_all_comm``,
``reduce_forward`` / ``reduce_backward`` inside ``Linear1D_Col/Row``; call sites
cornstarch/shardformer/modeling/llama.py:164-167,447-452,507-511 and
cornstarch/shardformer/layers/operation.py:28-118).  They work on any backend (gloo on CPU, NCCL on
GPU); uneven shards along the gather dimension are supported because context parallelism hands ranks
token sets of different sizes.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def _world(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


class _AllReduceFwd(torch.autograd.Function):
    """all-reduce in forward, identity in backward (output of a row-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllReduceBwd(torch.autograd.Function):
    """identity in forward, all-reduce in backward (input of a column-parallel linear)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllReduceSum(torch.autograd.Function):
    """all-reduce in forward AND backward (partial sums whose every rank consumes the total)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def reduce_forward(x, group):
    return x if _world(group) == 1 else _AllReduceFwd.apply(x, group)


def reduce_backward(x, group):
    return x if _world(group) == 1 else _AllReduceBwd.apply(x, group)


def all_reduce_sum_autograd(x, group):
    """Sum of per-rank partial values, each rank then using the total (gradient flows to the local partial)."""
    return x if _world(group) == 1 else _AllReduceSum.apply(x, group)


def all_gather_uneven(x: torch.Tensor, dim: int, group, sizes: list[int] | None = None):
    """All-gather along ``dim`` where ranks may hold different extents.  Returns ``(cat, sizes)``."""
    ws = _world(group)
    if ws == 1:
        return x, [x.shape[dim]]
    if sizes is None:
        mine = torch.tensor([x.shape[dim]], dtype=torch.int64, device=x.device)
        all_sizes = [torch.zeros_like(mine) for _ in range(ws)]
        dist.all_gather(all_sizes, mine, group=group)
        sizes = [int(s.item()) for s in all_sizes]
    x = x.contiguous()
    if len(set(sizes)) == 1:
        parts = [torch.empty_like(x) for _ in range(ws)]
        dist.all_gather(parts, x, group=group)
    else:
        # pad to the largest shard: plain all_gather works on every backend
        mx = max(sizes)
        pad_shape = list(x.shape)
        pad_shape[dim] = mx
        buf = x.new_zeros(pad_shape)
        buf.narrow(dim, 0, x.shape[dim]).copy_(x)
        padded = [torch.empty_like(buf) for _ in range(ws)]
        dist.all_gather(padded, buf, group=group)
        parts = [p.narrow(dim, 0, s) for p, s in zip(padded, sizes)]
    return torch.cat(parts, dim=dim), sizes


class _GatherFwdSplitBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group, grad_scale):
        out, sizes = all_gather_uneven(x, dim, group)
        ctx.dim, ctx.group, ctx.sizes, ctx.grad_scale = dim, group, sizes, grad_scale
        return out

    @staticmethod
    def backward(ctx, g):
        rank = dist.get_rank(ctx.group)
        start = sum(ctx.sizes[:rank])
        piece = g.narrow(ctx.dim, start, ctx.sizes[rank])
        if ctx.grad_scale is not None:
            piece = piece * ctx.grad_scale
        return piece.contiguous(), None, None, None


class _SplitFwdGatherBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group, grad_scale):
        ws, rank = dist.get_world_size(group), dist.get_rank(group)
        ctx.dim, ctx.group, ctx.grad_scale = dim, group, grad_scale
        chunks = torch.tensor_split(x, ws, dim=dim)
        ctx.sizes = [c.shape[dim] for c in chunks]
        return chunks[rank].contiguous()

    @staticmethod
    def backward(ctx, g):
        if ctx.grad_scale is not None:
            g = g * ctx.grad_scale
        out, _ = all_gather_uneven(g, ctx.dim, ctx.group, ctx.sizes)
        return out, None, None, None


def gather_forward_split_backward(x, dim: int, group, grad_scale: float | None = None):
    """Uneven all-gather along ``dim`` in forward; keep my slice (times ``grad_scale``) in backward."""
    return x if _world(group) == 1 else _GatherFwdSplitBwd.apply(x, dim, group, grad_scale)


def split_forward_gather_backward(x, dim: int, group, grad_scale: float | None = None):
    """Keep my ``tensor_split`` chunk along ``dim`` in forward; all-gather the gradient in backward."""
    return x if _world(group) == 1 else _SplitFwdGatherBwd.apply(x, dim, group, grad_scale)


class _AllToAll(torch.autograd.Function):
    """Ulysses exchange: scatter ``scatter_dim`` across the group, gather ``gather_dim``."""

    @staticmethod
    def forward(ctx, x, scatter_dim, gather_dim, group):
        ctx.scatter_dim, ctx.gather_dim, ctx.group = scatter_dim, gather_dim, group
        return _all_to_all(x, scatter_dim, gather_dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g, ctx.gather_dim, ctx.scatter_dim, ctx.group), None, None, None


def _all_to_all(x, scatter_dim, gather_dim, group):
    ws = dist.get_world_size(group)
    ins = [t.contiguous() for t in torch.tensor_split(x, ws, dim=scatter_dim)]
    if dist.get_backend(group) == "gloo":
        # gloo has no all_to_all: every rank gathers everything and keeps its column
        rank = dist.get_rank(group)
        stacked = torch.stack(ins, dim=0)
        everyone = [torch.empty_like(stacked) for _ in range(ws)]
        dist.all_gather(everyone, stacked, group=group)
        outs = [everyone[src][rank] for src in range(ws)]
    else:
        outs = [torch.empty_like(ins[0]) for _ in range(ws)]
        dist.all_to_all(outs, ins, group=group)
    return torch.cat(outs, dim=gather_dim)


def all_to_all_comm(x, group, scatter_dim: int = 2, gather_dim: int = 1):
    """``[B, S/sp, H] <-> [B, S, H/sp]`` exchange of Ulysses sequence parallelism (equal shards)."""
    return x if _world(group) == 1 else _AllToAll.apply(x, scatter_dim, gather_dim, group)


def reduce_scatter_uneven(x: torch.Tensor, dim: int, group, sizes: list[int]) -> torch.Tensor:
    """Sum ``x`` over the group and return this rank's slice of ``dim`` (slices may differ in size)."""
    ws, rank = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    if dist.get_backend(group) != "gloo" and len(set(sizes)) == 1 and dim == 0:
        out = torch.empty((sizes[0], *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, group=group)
        return out
    if dist.get_backend(group) != "gloo":
        # pad every rank's slice to the largest one so that a plain reduce_scatter applies
        mx = max(sizes)
        chunks, start = [], 0
        for s in sizes:
            c = x.narrow(dim, start, s)
            if s < mx:
                pad_shape = list(c.shape)
                pad_shape[dim] = mx - s
                c = torch.cat([c, c.new_zeros(pad_shape)], dim=dim)
            chunks.append(c.contiguous())
            start += s
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=group)
        return out.narrow(dim, 0, sizes[rank]).contiguous()
    dist.all_reduce(x, group=group)
    return x.narrow(dim, sum(sizes[:rank]), sizes[rank]).contiguous()


class _GatherFwdReduceScatterBwd(torch.autograd.Function):
    """All-gather (uneven) in forward, reduce-scatter of the gradient in backward: K/V under context parallelism."""

    @staticmethod
    def forward(ctx, x, dim, group, sizes):
        out, sizes = all_gather_uneven(x, dim, group, sizes)
        ctx.dim, ctx.group, ctx.sizes = dim, group, sizes
        return out

    @staticmethod
    def backward(ctx, g):
        return reduce_scatter_uneven(g, ctx.dim, ctx.group, ctx.sizes), None, None, None


def gather_forward_reduce_scatter_backward(x, dim: int, group, sizes: list[int] | None = None):
    return x if _world(group) == 1 else _GatherFwdReduceScatterBwd.apply(x, dim, group, sizes)


def _shift(send: torch.Tensor | None, recv: torch.Tensor | None, group, to_next: bool) -> None:
    """One neighbour exchange along the group's rank order: ``send`` goes to the next (previous) rank, ``recv`` is filled
    by the previous (next) one.  Ranks at the ends pass ``None`` for the side they do not have."""
    rank = dist.get_rank(group)
    ops = []
    if send is not None:
        ops.append(dist.P2POp(dist.isend, send, dist.get_global_rank(group, rank + (1 if to_next else -1)), group))
    if recv is not None:
        ops.append(dist.P2POp(dist.irecv, recv, dist.get_global_rank(group, rank - (1 if to_next else -1)), group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


class _HaloFromPrevious(torch.autograd.Function):
    """Prepend the last ``width`` entries (along ``dim``) of the previous rank's tensor; rank 0 prepends zeros.
    Backward returns the halo's gradient to the rank it came from, which adds it to its tail."""

    @staticmethod
    def forward(ctx, x, dim, width, group):
        ws, rank = dist.get_world_size(group), dist.get_rank(group)
        assert x.shape[dim] >= width, "a sequence shard is shorter than the halo of the convolution"
        ctx.dim, ctx.width, ctx.group = dim, width, group
        shape = list(x.shape)
        shape[dim] = width
        halo = x.new_zeros(shape)
        tail = x.narrow(dim, x.shape[dim] - width, width).contiguous() if rank < ws - 1 else None
        _shift(tail, halo if rank > 0 else None, group, to_next=True)
        return torch.cat([halo, x], dim=dim)

    @staticmethod
    def backward(ctx, g):
        dim, width, group = ctx.dim, ctx.width, ctx.group
        ws, rank = dist.get_world_size(group), dist.get_rank(group)
        gx = g.narrow(dim, width, g.shape[dim] - width).clone()
        g_halo = g.narrow(dim, 0, width).contiguous() if rank > 0 else None
        from_next = torch.empty_like(g.narrow(dim, 0, width)).contiguous() if rank < ws - 1 else None
        _shift(g_halo, from_next, group, to_next=False)
        if from_next is not None:
            gx.narrow(dim, gx.shape[dim] - width, width).add_(from_next)
        return gx, None, None, None


def halo_from_previous(x, dim: int, width: int, group):
    """``[previous rank's last width entries | x]`` along ``dim``: the left context of a causal convolution over a
    sequence that is split in contiguous chunks in rank order."""
    if _world(group) == 1 or width == 0:
        shape = list(x.shape)
        shape[dim] = width
        return torch.cat([x.new_zeros(shape), x], dim=dim)
    return _HaloFromPrevious.apply(x, dim, width, group)
