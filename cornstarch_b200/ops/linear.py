"""Linear layers on the tcgen05 GEMM with gradient-accumulation fusion.

``linear(x, weight, bias)`` is ``F.linear`` with a custom backward made of two more native GEMMs.
When a weight carries a ``main_grad`` attribute (a view into the engine's flat gradient buffer,
see :mod:`cornstarch_b200.optim.arena`) the weight gradient is accumulated straight into it by the
GEMM epilogue and autograd receives ``None`` for that weight; otherwise a normal gradient is
returned.

``multi_linear(x, weights, biases)`` runs several projections of the same input (q/k/v, gate/up) as
ONE GEMM when the weights sit back to back in memory (which the arena guarantees), and falls back to
one GEMM per weight otherwise.  The output is the concatenation along the last dimension.

Replaces ``nn.Linear`` / ``Linear1D_Col`` / ``Linear1D_Row`` / ``FusedLinear1D_Col`` used by the
reference policies (cornstarch/shardformer/policies/llama.py:192-249, policies/phi3.py:181-208).
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.nn.functional as F

from . import _native as nat
from .gemm import gemm


def _use_native(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not nat.LIBRARY_MODE


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


def colsum(x2: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """Column sums of a bf16 ``[rows, H]`` matrix (bias gradients) on the native kernel."""
    rows, H = x2.shape
    if not _use_native(x2) or H % 8 or not x2.is_contiguous():
        s = x2.float().sum(0)
        if out is None:
            return s.to(x2.dtype)
        out.copy_((out.float() + s if accumulate else s).to(out.dtype))
        return out
    if out is None:
        out = torch.empty(H, dtype=x2.dtype, device=x2.device)
        accumulate = False
    parts = nat.lib().csb_colsum_parts(rows)
    scratch = torch.empty(parts * H, dtype=torch.float32, device=x2.device)
    nat.check(
        nat.lib().csb_colsum(x2.data_ptr(), scratch.data_ptr(), out.data_ptr(), int(out.dtype == torch.float32),
                             int(accumulate), rows, H, nat.stream()),
        "csb_colsum",
    )
    return out


def fuse_adjacent(tensors: Sequence[torch.Tensor]) -> torch.Tensor | None:
    """If 2-D row-major tensors with equal width sit back to back in one storage, return the stacked view."""
    t0 = tensors[0]
    if any(t.dim() != 2 or not t.is_contiguous() or t.shape[1] != t0.shape[1] or t.dtype != t0.dtype for t in tensors):
        return None
    end = t0.data_ptr() + t0.numel() * t0.element_size()
    rows = t0.shape[0]
    for t in tensors[1:]:
        if t.data_ptr() != end or t.untyped_storage().data_ptr() != t0.untyped_storage().data_ptr():
            return None
        end += t.numel() * t.element_size()
        rows += t.shape[0]
    return torch.as_strided(t0, (rows, t0.shape[1]), (t0.shape[1], 1), t0.storage_offset())


def fuse_adjacent_1d(tensors: Sequence[torch.Tensor | None]) -> torch.Tensor | None:
    if any(t is None for t in tensors):
        return None
    t0 = tensors[0]
    end = t0.data_ptr() + t0.numel() * t0.element_size()
    n = t0.numel()
    for t in tensors[1:]:
        if t.data_ptr() != end or t.untyped_storage().data_ptr() != t0.untyped_storage().data_ptr():
            return None
        end += t.numel() * t.element_size()
        n += t.numel()
    return torch.as_strided(t0, (n,), (1,), t0.storage_offset())


class _LinearFn(torch.autograd.Function):
    """y = x W^T + b with native backward; several (weight, bias) pairs share one input."""

    @staticmethod
    def forward(ctx, x, n_w, act, tp, *params):
        weights = params[:n_w]
        biases = params[n_w:]
        x2 = _as_2d(x)
        ctx.tp = tp
        fused_w = fuse_adjacent(weights) if n_w > 1 else weights[0]
        has_bias = biases[0] is not None
        fused_b = (fuse_adjacent_1d(biases) if n_w > 1 else biases[0]) if has_bias else None
        n_total = sum(w.shape[0] for w in weights)
        # the returned tensor owns its storage (callers such as RoPE modify it in place)
        out = torch.empty((*x.shape[:-1], n_total), dtype=x.dtype, device=x.device)
        y = out.view(-1, n_total)
        assert not (tp is not None and tp[0] == "row" and (has_bias or n_w != 1)), "row-parallel: one weight, bias added after the reduce"
        if tp is not None and tp[0] == "row" and fused_w is not None and not has_bias:
            # row-parallel: partial products of all ranks are summed by the fused GEMM + all-reduce kernel
            tp[1].gemm_allreduce(x2, fused_w, out=y)
        elif fused_w is not None and (not has_bias or fused_b is not None):
            gemm(x2, fused_w, bias=fused_b, act=act, out=y)
        else:
            o = 0
            for w, b in zip(weights, biases):
                gemm(x2, w, bias=b, act=act, out=y[:, o : o + w.shape[0]])
                o += w.shape[0]
        ctx.save_for_backward(x2, *weights)
        ctx.n_w = n_w
        ctx.has_bias = has_bias
        ctx.x_shape = x.shape
        ctx.biases = biases
        assert act is None, "activation epilogues are applied outside autograd-tracked linears"
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, *weights = ctx.saved_tensors
        n_w = ctx.n_w
        dy2 = _as_2d(dy)
        fused_w = fuse_adjacent(weights) if n_w > 1 else weights[0]
        dx = None
        if ctx.needs_input_grad[0]:
            if fused_w is not None and ctx.tp is not None and ctx.tp[0] == "col":
                # column-parallel: dx is a partial sum over the output shards -> fused GEMM + all-reduce
                dx = ctx.tp[1].gemm_allreduce(dy2, fused_w, b_mn_major=True)
            elif fused_w is not None:
                dx = gemm(dy2, fused_w, b_mn_major=True)
            else:
                o = 0
                dx = torch.empty_like(x2)
                for i, w in enumerate(weights):
                    gemm(dy2[:, o : o + w.shape[0]], w, b_mn_major=True, out=dx, accumulate=i > 0)
                    o += w.shape[0]
                if ctx.tp is not None and ctx.tp[0] == "col":
                    # weights not adjacent in memory (no parameter arena): plain GEMMs, then the NCCL all-reduce
                    import torch.distributed as dist

                    dist.all_reduce(dx, group=ctx.tp[1].group)
            dx = dx.view(ctx.x_shape)
        dws: list = [None] * n_w
        dbs: list = [None] * n_w
        need_w = [ctx.needs_input_grad[4 + i] for i in range(n_w)]
        if any(need_w):
            mains = [getattr(w, "main_grad", None) for w in weights]
            fused_main = None
            if all(m is not None for m in mains):
                fused_main = fuse_adjacent(mains) if n_w > 1 else mains[0]
            if fused_main is not None and fused_w is not None:
                # one GEMM accumulating into the flat gradient buffer
                gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=fused_main, accumulate=True)
                for w in weights:
                    w.grad_added_to_main_grad = True
            else:
                o = 0
                for i, w in enumerate(weights):
                    n = w.shape[0]
                    if need_w[i]:
                        if mains[i] is not None:
                            gemm(dy2[:, o : o + n], x2, a_mn_major=True, b_mn_major=True, out=mains[i], accumulate=True)
                            w.grad_added_to_main_grad = True
                        else:
                            dws[i] = gemm(dy2[:, o : o + n], x2, a_mn_major=True, b_mn_major=True)
                    o += n
        if ctx.has_bias:
            o = 0
            for i, (w, b) in enumerate(zip(weights, ctx.biases)):
                n = w.shape[0]
                if ctx.needs_input_grad[4 + n_w + i]:
                    seg = dy2[:, o : o + n]
                    main = getattr(b, "main_grad", None)
                    if main is not None:
                        colsum(seg.contiguous() if not seg.is_contiguous() else seg, out=main, accumulate=True)
                        b.grad_added_to_main_grad = True
                    else:
                        dbs[i] = colsum(seg.contiguous() if not seg.is_contiguous() else seg)
                o += n
        return (dx, None, None, None, *dws, *dbs)


def multi_linear(x: torch.Tensor, weights: Sequence[torch.Tensor], biases: Sequence[torch.Tensor | None] | None = None,
                 tp=None):
    """Concatenated projections ``[x W_0^T + b_0 | x W_1^T + b_1 | ...]`` of one input.

    ``tp = ("col" | "row", FusedTensorParallel)`` fuses the tensor-parallel all-reduce into the GEMM: for a
    row-parallel weight in the forward, for column-parallel weights in the input-gradient GEMM of the backward.
    """
    if biases is None:
        biases = [None] * len(weights)
    if not _use_native(x):
        assert tp is None
        outs = [F.linear(x, w, b) for w, b in zip(weights, biases)]
        return outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)
    return _LinearFn.apply(x, len(weights), None, tp, *weights, *biases)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, tp=None) -> torch.Tensor:
    return multi_linear(x, [weight], [bias], tp)


# ------------------------------------------------------------------------------------------------ grouped (per-expert) linears
class _GroupedLinearFn(torch.autograd.Function):
    """``y[g] = x[g] [W_g0 | W_g1 | ...]^T`` for every group ``g`` of ``group_rows`` rows: the forward GEMMs of all groups are
    one launch and so are the input-gradient GEMMs (``ops.gemm.grouped_gemm``); the weight gradients are one GEMM per
    group, accumulated into ``main_grad`` where the weight has one."""

    @staticmethod
    def forward(ctx, x2, group_rows, n_w, *weights):
        G = len(weights) // n_w
        groups = [weights[g * n_w : (g + 1) * n_w] for g in range(G)]
        from .gemm import grouped_gemm

        widths = [w.shape[0] for w in groups[0]]
        out = torch.empty((x2.shape[0], sum(widths)), dtype=x2.dtype, device=x2.device)
        fused = [fuse_adjacent(ws) if n_w > 1 else ws[0] for ws in groups]
        if all(f is not None for f in fused):
            grouped_gemm(x2, fused, group_rows, out=out)
        else:
            o = 0
            for j, n in enumerate(widths):
                grouped_gemm(x2, [ws[j] for ws in groups], group_rows, out=out[:, o : o + n])
                o += n
        ctx.save_for_backward(x2, *weights)
        ctx.group_rows, ctx.n_w, ctx.widths = group_rows, n_w, widths
        return out

    @staticmethod
    def backward(ctx, dy):
        from .gemm import grouped_gemm

        x2, *weights = ctx.saved_tensors
        R, n_w, widths = ctx.group_rows, ctx.n_w, ctx.widths
        G = len(weights) // n_w
        groups = [weights[g * n_w : (g + 1) * n_w] for g in range(G)]
        dy2 = _as_2d(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            fused = [fuse_adjacent(ws) if n_w > 1 else ws[0] for ws in groups]
            if all(f is not None for f in fused):
                dx = grouped_gemm(dy2, fused, R, b_mn_major=True)
            else:
                dx = torch.empty_like(x2)
                o = 0
                for j, n in enumerate(widths):
                    grouped_gemm(dy2[:, o : o + n], [ws[j] for ws in groups], R, b_mn_major=True, out=dx, accumulate=j > 0)
                    o += n
        dws: list = []
        for g, ws in enumerate(groups):
            rows = slice(g * R, (g + 1) * R)
            need = [ctx.needs_input_grad[3 + g * n_w + j] for j in range(n_w)]
            dws += _weight_grads(dy2[rows], x2[rows], ws, need)
        return (dx, None, None, *dws)


def grouped_multi_linear(x2: torch.Tensor, weight_groups: Sequence[Sequence[torch.Tensor]], group_rows: int) -> torch.Tensor:
    """Bias-free projections of a row-grouped input: rows ``[g * group_rows, (g + 1) * group_rows)`` of ``x2`` are
    multiplied with the weights of group ``g`` (``weight_groups[g]``, e.g. ``[w1, w3]`` of expert ``g``; every group has
    the same shapes), outputs concatenated along the last dimension as ``multi_linear`` does."""
    G = len(weight_groups)
    assert x2.dim() == 2 and x2.shape[0] == G * group_rows
    n_w = len(weight_groups[0])
    if not _use_native(x2):
        outs = []
        for g, ws in enumerate(weight_groups):
            seg = x2[g * group_rows : (g + 1) * group_rows]
            outs.append(torch.cat([F.linear(seg, w) for w in ws], dim=-1) if n_w > 1 else F.linear(seg, ws[0]))
        return torch.cat(outs, dim=0)
    flat = [w for ws in weight_groups for w in ws]
    return _GroupedLinearFn.apply(_as_2d(x2), group_rows, n_w, *flat)


# ------------------------------------------------------------------------------------------------ sequence-sharded TP
# Activations between the tensor-parallel blocks are sharded by token rows (rank r holds a contiguous range of whole
# 128-row tiles): norms, residual adds and everything token-wise run on 1/tp of the tokens.  A column-parallel
# projection gathers its input inside the GEMM (all-gather -> GEMM), a row-parallel one scatters its output inside
# the GEMM (GEMM -> reduce-scatter); the backward passes use the same two kernels with the roles swapped.  On CUDA both
# are single kernels over peer memory (parallel/symm.py); elsewhere torch.distributed collectives state the same math.
def _gather_rows(x2: torch.Tensor, group) -> torch.Tensor:
    import torch.distributed as dist

    ws = dist.get_world_size(group)
    parts = [torch.empty_like(x2) for _ in range(ws)]
    dist.all_gather(parts, x2.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def _scatter_rows_sum(y2: torch.Tensor, group) -> torch.Tensor:
    import torch.distributed as dist

    ws, r = dist.get_world_size(group), dist.get_rank(group)
    y2 = y2.contiguous()
    dist.all_reduce(y2, group=group)
    rows = y2.shape[0] // ws
    return y2[r * rows : (r + 1) * rows].clone()


class _AgLinearFn(torch.autograd.Function):
    """``y = all_gather_rows(x_shard) [W_0; W_1; ...]^T``: column-parallel projections of a row-sharded input."""

    @staticmethod
    def forward(ctx, x_shard, group, ftp, n_w, *weights):
        x2 = _as_2d(x_shard)
        fused_w = fuse_adjacent(weights) if n_w > 1 else weights[0]
        if ftp is not None and fused_w is not None:
            y, x_full = ftp.ag_gemm(x2, fused_w)
        else:
            x_full = _gather_rows(x2, group)
            if _use_native(x_full) and fused_w is not None:
                y = gemm(x_full, fused_w)
            else:
                y = torch.cat([F.linear(x_full, w) for w in weights], dim=-1)
        ctx.save_for_backward(x_full, *weights)
        ctx.group, ctx.ftp, ctx.n_w, ctx.x_shape = group, ftp, n_w, x_shard.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, *weights = ctx.saved_tensors
        n_w = ctx.n_w
        dy2 = _as_2d(dy)
        fused_w = fuse_adjacent(weights) if n_w > 1 else weights[0]
        dx = None
        if ctx.needs_input_grad[0]:
            if ctx.ftp is not None and fused_w is not None:
                dx = ctx.ftp.gemm_reducescatter(dy2, fused_w, b_mn_major=True)  # partial sums over the output shards
            else:
                full = dy2.float() @ torch.cat([w.float() for w in weights], dim=0)
                dx = _scatter_rows_sum(full.to(dy.dtype), ctx.group)
            dx = dx.view(ctx.x_shape)
        dws = _weight_grads(dy2, x_full, weights, [ctx.needs_input_grad[4 + i] for i in range(n_w)])
        return (dx, None, None, None, *dws)


class _RsLinearFn(torch.autograd.Function):
    """``y_shard = reduce_scatter_rows(x W^T)``: a row-parallel projection whose output is row-sharded."""

    @staticmethod
    def forward(ctx, x, group, ftp, weight):
        x2 = _as_2d(x)
        if ftp is not None:
            y = ftp.gemm_reducescatter(x2, weight)
        else:
            y = _scatter_rows_sum(gemm(x2, weight) if _use_native(x2) else F.linear(x2, weight), group)
        ctx.save_for_backward(x2, weight)
        ctx.group, ctx.ftp, ctx.x_shape = group, ftp, x.shape
        return y

    @staticmethod
    def backward(ctx, dy_shard):
        x2, weight = ctx.saved_tensors
        dy2 = _as_2d(dy_shard)
        if ctx.ftp is not None:
            dx, dy_full = ctx.ftp.ag_gemm(dy2, weight, b_mn_major=True)  # dx = all_gather(dy) W
        else:
            dy_full = _gather_rows(dy2, ctx.group)
            dx = gemm(dy_full, weight, b_mn_major=True) if _use_native(dy_full) else dy_full @ weight
        dws = _weight_grads(dy_full, x2, [weight], [ctx.needs_input_grad[3]])
        return dx.view(ctx.x_shape) if ctx.needs_input_grad[0] else None, None, None, dws[0]


def _offsets(weights):
    o = 0
    for w in weights:
        yield o, w
        o += w.shape[0]


def _weight_grads(dy2, x2, weights, need):
    """``dW_i = dy_i^T x`` for every weight: accumulated into ``main_grad`` when the weight has one (autograd then gets
    ``None``), returned otherwise."""
    dws = [None] * len(weights)
    if not any(need):
        return dws
    native = _use_native(dy2)
    mains = [getattr(w, "main_grad", None) for w in weights]
    fused_main = None
    if native and all(m is not None for m in mains):
        fused_main = fuse_adjacent(mains) if len(weights) > 1 else mains[0]
    if fused_main is not None and (len(weights) == 1 or fuse_adjacent(weights) is not None):
        gemm(dy2, x2, a_mn_major=True, b_mn_major=True, out=fused_main, accumulate=True)
        for w in weights:
            w.grad_added_to_main_grad = True
        return dws
    for i, (o, w) in enumerate(_offsets(weights)):
        if not need[i]:
            continue
        seg = dy2[:, o : o + w.shape[0]]
        if native and mains[i] is not None:
            gemm(seg, x2, a_mn_major=True, b_mn_major=True, out=mains[i], accumulate=True)
            w.grad_added_to_main_grad = True
        elif native:
            dws[i] = gemm(seg, x2, a_mn_major=True, b_mn_major=True)
        else:
            dws[i] = (seg.float().t() @ x2.float()).to(w.dtype)
    return dws


def ag_linear(x_shard: torch.Tensor, weights: Sequence[torch.Tensor], group, ftp=None) -> torch.Tensor:
    """Column-parallel projections (no bias) of a row-sharded input: returns ``[rows * tp, sum of local widths]``."""
    return _AgLinearFn.apply(x_shard, group, ftp, len(weights), *weights)


def rs_linear(x: torch.Tensor, weight: torch.Tensor, group, ftp=None) -> torch.Tensor:
    """Row-parallel projection (no bias) with a row-sharded output: returns ``[rows / tp, out]``."""
    return _RsLinearFn.apply(x, group, ftp, weight)


def add_adapter_deltas(y: torch.Tensor, x: torch.Tensor, projections) -> torch.Tensor:
    """``y`` = fused output of several projections of ``x`` (concatenated on the last dim).  Projections that carry an
    adapter (a ``delta(x)`` method returning their additive update, e.g. LoRA) get it added to their slice."""
    if not any(hasattr(p, "delta") for p in projections):
        return y
    parts, lo = [], 0
    for p in projections:
        n = p.weight.shape[0]
        piece = y[..., lo : lo + n]
        if hasattr(p, "delta"):
            piece = piece + p.delta(x)
        parts.append(piece)
        lo += n
    return torch.cat(parts, dim=-1)
