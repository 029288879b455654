"""Fused LM-head + cross-entropy that never materialises the full ``[tokens, vocab]`` logits.

``linear_cross_entropy(hidden, weight, labels)`` walks the tokens in chunks: logits chunk on the
tcgen05 GEMM, per-row max / sum-exp / target logit (``ce_stats``), and — in the backward — the
softmax-minus-onehot gradient written in place over the logits chunk (``ce_grad``) followed by the two
gradient GEMMs.  Between forward and backward ``3 * tokens`` floats are kept and, when they fit a budget
(``CORNSTARCH_B200_CE_KEEP_LOGITS_GB``, default 4 GiB), the bf16 logits themselves: the loss's backward follows its
forward immediately, so the buffer lives for a moment and saves the recomputation of the largest GEMM of the model
(2 * tokens * vocab * hidden FLOPs per micro-batch).  Larger problems recompute the logits chunk by chunk.

With a tensor-parallel group the weight is a vocab shard ``[V/tp, H]`` starting at ``vocab_start``; the
row statistics are combined with three small all-reduces (max, rescaled sum, target logit), which is
the ``dist_cross_entropy`` contract of the reference
(cornstarch/shardformer/modeling/llama.py:379-392).  Labels are NOT shifted here.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import _native as nat
from .gemm import gemm


KEEP_LOGITS_BYTES = int(float(os.environ.get("CORNSTARCH_B200_CE_KEEP_LOGITS_GB", "4")) * 2**30)


def cross_entropy_reference(hidden, weight, labels, ignore_index=-100):
    logits = F.linear(hidden.float(), weight.float())
    return F.cross_entropy(logits, labels, ignore_index=ignore_index, reduction="sum"), (labels != ignore_index).sum()


def _stats(logits, labels, vocab_start):
    rows, V = logits.shape
    mx = torch.empty(rows, dtype=torch.float32, device=logits.device)
    sm = torch.empty_like(mx)
    tg = torch.empty_like(mx)
    nat.check(
        nat.lib().csb_ce_stats(logits.data_ptr(), logits.stride(0), labels.data_ptr(), V, vocab_start, mx.data_ptr(),
                               sm.data_ptr(), tg.data_ptr(), rows, nat.stream()),
        "csb_ce_stats",
    )
    return mx, sm, tg


def _combine_tp(mx, sm, tg, group):
    if group is None or dist.get_world_size(group) == 1:
        return mx, sm, tg
    gmx = mx.clone()
    dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=group)
    sm = sm * torch.exp(mx - gmx)
    dist.all_reduce(sm, group=group)
    dist.all_reduce(tg, group=group)
    return gmx, sm, tg


class _LinearCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index, chunk, group, vocab_start, keep_logits):
        T, H = hidden.shape
        V = weight.shape[0]
        labels = labels.contiguous()
        loss_sum = torch.zeros((), dtype=torch.float32, device=hidden.device)
        row_max = torch.empty(T, dtype=torch.float32, device=hidden.device)
        row_sum = torch.empty_like(row_max)
        row_tgt = torch.empty_like(row_max)
        keep = keep_logits if keep_logits is not None else (T * V * hidden.element_size() <= KEEP_LOGITS_BYTES)
        keep = keep and (ctx.needs_input_grad[0] or ctx.needs_input_grad[1])
        buf = torch.empty((T if keep else min(chunk, T), V), dtype=hidden.dtype, device=hidden.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = buf[s:e] if keep else buf[: e - s]
            gemm(hidden[s:e], weight, out=lg)
            mx, sm, tg = _stats(lg, labels[s:e], vocab_start)
            mx, sm, tg = _combine_tp(mx, sm, tg, group)
            row_max[s:e], row_sum[s:e], row_tgt[s:e] = mx, sm, tg
        valid = labels != ignore_index
        per_row = torch.log(row_sum) + row_max - row_tgt
        loss_sum = torch.where(valid, per_row, torch.zeros_like(per_row)).sum()
        ctx.save_for_backward(hidden, weight, labels, row_max, row_sum, row_tgt)
        ctx.args = (ignore_index, chunk, group, vocab_start)
        ctx.logits = buf if keep else None  # overwritten with the gradient by the first backward pass
        return loss_sum

    @staticmethod
    def backward(ctx, go):
        hidden, weight, labels, row_max, row_sum, row_tgt = ctx.saved_tensors
        ignore_index, chunk, group, vocab_start = ctx.args
        T, H = hidden.shape
        V = weight.shape[0]
        scale = go.reshape(1).float().contiguous()
        dh = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        main = getattr(weight, "main_grad", None)
        dW = None
        if ctx.needs_input_grad[1]:
            dW = main if main is not None else torch.zeros(weight.shape, dtype=torch.float32, device=hidden.device)
        kept, ctx.logits = ctx.logits, None  # a second backward pass (retain_graph) recomputes
        buf = kept if kept is not None else torch.empty((min(chunk, T), V), dtype=hidden.dtype, device=hidden.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            if kept is not None:
                lg = buf[s:e]
            else:
                lg = buf[: e - s]
                gemm(hidden[s:e], weight, out=lg)
            nat.check(
                nat.lib().csb_ce_grad(lg.data_ptr(), lg.stride(0), labels[s:e].data_ptr(), V, vocab_start,
                                      row_max[s:e].data_ptr(), row_sum[s:e].data_ptr(), row_tgt[s:e].data_ptr(), None,
                                      scale.data_ptr(), ignore_index, e - s, nat.stream()),
                "csb_ce_grad",
            )
            if dh is not None:
                gemm(lg, weight, b_mn_major=True, out=dh[s:e])
            if dW is not None:
                gemm(lg, hidden[s:e], a_mn_major=True, b_mn_major=True, out=dW, accumulate=True)
        dw_ret = None
        if dW is not None:
            if main is not None:
                weight.grad_added_to_main_grad = True
            else:
                dw_ret = dW.to(weight.dtype)
        return dh, dw_ret, None, None, None, None, None, None


def linear_cross_entropy(hidden, weight, labels, ignore_index: int = -100, chunk: int = 4096, tp_group=None,
                         vocab_start: int = 0, reduction: str = "mean", keep_logits: bool | None = None):
    """Cross-entropy of ``hidden @ weight.T`` against ``labels`` (already aligned with the rows of ``hidden``).

    ``hidden``: ``[..., H]``; ``weight``: ``[V_local, H]``; ``labels``: ``[...]`` int64 with ``ignore_index`` rows
    skipped.  ``reduction``: ``"mean"`` over valid rows, ``"sum"``, or ``"sum_and_count"`` (returns both, for
    callers that normalise across micro-batches or sequence-parallel ranks themselves).  ``keep_logits``: keep the
    bf16 logits for the backward pass instead of recomputing them (``None``: when they fit ``KEEP_LOGITS_BYTES``).
    """
    H = hidden.shape[-1]
    h2 = hidden.reshape(-1, H)
    lab = labels.reshape(-1)
    n_valid = (lab != ignore_index).sum()
    if hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0 and not nat.LIBRARY_MODE:
        h2 = h2 if h2.is_contiguous() else h2.contiguous()
        loss_sum = _LinearCEFn.apply(h2, weight, lab, ignore_index, chunk, tp_group, vocab_start, keep_logits)
    else:
        loss_sum = _ce_torch(h2, weight, lab, ignore_index, tp_group, vocab_start)
    if reduction == "sum":
        return loss_sum
    if reduction == "sum_and_count":
        return loss_sum, n_valid
    return loss_sum / n_valid.clamp(min=1).to(loss_sum.dtype)


def _ce_torch(h2, weight, lab, ignore_index, group, vocab_start):
    """PyTorch path (CPU / fp32), vocab-parallel aware through differentiable all-reduces."""
    logits = F.linear(h2, weight).float()
    if group is None or dist.get_world_size(group) == 1:
        return F.cross_entropy(logits, lab, ignore_index=ignore_index, reduction="sum")
    from ..parallel.comm import all_reduce_sum_autograd

    V = weight.shape[0]
    mx = logits.detach().max(dim=-1).values
    dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=group)
    ex = torch.exp(logits - mx[:, None])
    sm = all_reduce_sum_autograd(ex.sum(-1), group)
    local = lab - vocab_start
    inside = (local >= 0) & (local < V)
    tgt = torch.gather(logits, 1, local.clamp(0, V - 1)[:, None])[:, 0]
    tgt = all_reduce_sum_autograd(torch.where(inside, tgt, torch.zeros_like(tgt)), group)
    per_row = torch.log(sm) + mx - tgt
    valid = lab != ignore_index
    return torch.where(valid, per_row, torch.zeros_like(per_row)).sum()
