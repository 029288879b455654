"""Activation recomputation of a transformer layer that keeps the attention output.

``checkpoint_layer(fn, *args)`` behaves like ``torch.utils.checkpoint.checkpoint``: the layer's activations are
dropped after the forward pass and rebuilt in the backward pass.  The difference is that the attention output and
its log-sum-exp are kept (:class:`cornstarch_b200.ops.attention.attention_tape`), so the recomputation skips the
flash-attention forward kernel, whose cost grows with the square of the sequence length while the kept tensors
grow linearly.  The reference enables plain non-reentrant checkpointing on every sub-model
(cornstarch/models/multimodal_language_model/modeling_multimodal_language_model.py:774-792).

Arguments that are not tensors (masks, ``None``) and tuples of tensors (rotary tables) pass through unchanged;
only top-level tensor arguments are differentiated.  The layer may return a tensor or a tuple with ``None`` entries.
"""

from __future__ import annotations

import torch

from ..ops.attention import attention_tape


class _Recompute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run, anchor, *tensors):
        tape: list = []
        with torch.no_grad(), attention_tape(tape, "record"):
            outs = run(tensors)
        ctx.run, ctx.tape = run, tape
        ctx.req = [t.requires_grad for t in tensors]
        ctx.save_for_backward(*tensors)
        return outs

    @staticmethod
    def backward(ctx, *grads):
        tensors = [t.detach().requires_grad_(r) for t, r in zip(ctx.saved_tensors, ctx.req)]
        with torch.enable_grad(), attention_tape(ctx.tape, "replay"):
            outs = ctx.run(tensors)
        pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        ctx.tape = None
        return (None, None) + tuple(t.grad if r else None for t, r in zip(tensors, ctx.req))


def checkpoint_layer(fn, *args):
    """Run ``fn(*args)`` now without keeping activations; rebuild them (minus the attention forward) for backward."""
    idx = [i for i, a in enumerate(args) if isinstance(a, torch.Tensor)]
    tensors = [args[i] for i in idx]
    layout = {}

    def run(ts):
        full = list(args)
        for i, t in zip(idx, ts):
            full[i] = t
        out = fn(*full)
        single = not isinstance(out, (tuple, list))
        seq = (out,) if single else tuple(out)
        layout["single"] = single
        layout["none"] = [o is None for o in seq]
        return tuple(o for o in seq if o is not None)

    # parameters receive gradients inside backward(); the output must require grad even if no tensor input does
    anchor = torch.zeros((), requires_grad=True, device=tensors[0].device if tensors else None)
    outs = list(_Recompute.apply(run, anchor, *tensors))
    seq = [None if is_none else outs.pop(0) for is_none in layout["none"]]
    return seq[0] if layout["single"] else tuple(seq)
