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
import torch.distributed as dist

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


def activation_bytes_per_layer(cfg, tokens: int, tp: int = 1) -> int:
    """Upper estimate of what one dense decoder layer keeps for backward when it is not recomputed (bf16 activations):
    the inputs of both norms, the normed inputs of the projections, q / k / v after RoPE, the attention output, the
    gate-up output and the SwiGLU output."""
    H, I = cfg.hidden_size, cfg.intermediate_size
    D = getattr(cfg, "head_dim", None) or H // cfg.num_attention_heads
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * D
    return int(1.15 * tokens * 2 * (8 * H + (3 * qkv + 3 * I) / tp))


def tune_recompute(model, tokens: int, tp: int, in_flight: int, group=None, safety_bytes: int = 6 << 30) -> int:
    """After one fully recomputed step: how many decoder layers can keep their activations in the memory that step left
    free (what the driver still reports free; the caching allocator holds on to its peak).  The same number on every
    rank of ``group`` - the tensor-parallel peers replay the same collectives in a recomputed forward.  Returns the
    number of layers kept (0 for models this estimate does not cover)."""
    lm = getattr(model, "language_model", model)
    inner = getattr(lm, "model", None)
    cfg = getattr(lm, "config", None)
    keep = 0
    if torch.cuda.is_available() and inner is not None and hasattr(inner, "layers") and not getattr(cfg, "num_local_experts", 0):
        from ..models.base import is_released

        held = sum(not is_released(l) for l in inner.layers)
        torch.cuda.synchronize()
        free, _ = torch.cuda.mem_get_info()
        per_layer = activation_bytes_per_layer(cfg, tokens, tp) * max(in_flight, 1)
        keep = max(0, min(held, int((free - safety_bytes) // per_layer)))
    if group is not None and dist.get_world_size(group) > 1:
        t = torch.tensor([keep], device="cuda" if torch.cuda.is_available() else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
        keep = int(t)
    if inner is not None and hasattr(lm, "gradient_checkpointing_enable"):
        lm.gradient_checkpointing_enable({"keep_last_layers": keep})
    return keep


class RecomputeTuner:
    """Two passes of :func:`tune_recompute`, one after each of the first two steps.  The first uses the upper estimate of a
    layer's activations; the second replaces it by what the layers kept in step two actually cost (growth of the
    allocator's reservation per kept layer, plus 10 %, and never less than half the estimate) and keeps more layers if
    the memory the driver still reports free allows it."""

    def __init__(self, model, tokens: int, tp: int, in_flight: int, group=None, safety_bytes: int = 6 << 30):
        self.model, self.tokens, self.tp, self.in_flight = model, tokens, tp, max(in_flight, 1)
        self.group, self.safety = group, safety_bytes
        self.passes, self.keep, self.reserved0 = 0, 0, 0

    def after_step(self) -> int:
        self.passes += 1
        if self.passes == 1:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
                self.reserved0 = torch.cuda.memory_reserved()
            self.keep = tune_recompute(self.model, self.tokens, self.tp, self.in_flight, self.group, self.safety)
            return self.keep
        if self.passes > 2:
            return self.keep
        lm = getattr(self.model, "language_model", self.model)
        inner = getattr(lm, "model", None)
        extra = 0
        if torch.cuda.is_available() and inner is not None and self.keep > 0:
            from ..models.base import is_released

            held = sum(not is_released(l) for l in inner.layers)
            torch.cuda.synchronize()
            free, _ = torch.cuda.mem_get_info()
            estimate = activation_bytes_per_layer(lm.config, self.tokens, self.tp) * self.in_flight
            measured = (torch.cuda.memory_reserved() - self.reserved0) / self.keep
            per_layer = max(1.1 * measured, 0.5 * estimate)
            extra = max(0, min(held - self.keep, int((free - self.safety) // per_layer)))
        if self.group is not None and dist.get_world_size(self.group) > 1:
            t = torch.tensor([extra], device="cuda" if torch.cuda.is_available() else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
            extra = int(t)
        if extra > 0:
            self.keep += extra
            lm.gradient_checkpointing_enable({"keep_last_layers": self.keep})
        return self.keep
