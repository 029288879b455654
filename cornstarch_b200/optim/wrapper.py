"""Optimizer wrapper used by the plugins: ``backward`` / ``backward_by_grad`` / clipping / loss scaling.

Plays the role of ColossalAI's ``HybridParallelNaiveOptimizer`` / ``HybridParallelAMPOptimizer`` in the
reference (cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:627-654): fp16
uses a dynamic loss scale (``initial_scale=2**16``, growth x2 every ``growth_interval`` clean steps,
backoff x0.5 on overflow, bounded by ``min_scale`` / ``max_scale``); bf16 and fp32 use scale 1.  The global
gradient norm for clipping is summed over the tensor- and pipeline-parallel groups.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .fused_adamw import FusedAdamW


class DynamicLossScaler:
    def __init__(self, initial_scale=2.0**16, min_scale=1.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=1000,
                 hysteresis=2, max_scale=2.0**32):
        self.scale = float(initial_scale)
        self.min_scale, self.max_scale = float(min_scale), float(max_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval, self.hysteresis = growth_interval, hysteresis
        self._good, self._hyst = 0, hysteresis

    def update(self, overflow: bool) -> None:
        if overflow:
            self._hyst -= 1
            self._good = 0
            if self._hyst <= 0:
                self.scale = max(self.scale * self.backoff_factor, self.min_scale)
        else:
            self._good += 1
            if self._good % self.growth_interval == 0:
                self._hyst = self.hysteresis
                self.scale = min(self.scale * self.growth_factor, self.max_scale)


class OptimizerWrapper:
    def __init__(self, optim: torch.optim.Optimizer, model=None, max_norm: float = 0.0, precision: str | None = None,
                 tp_group=None, pp_group=None, scaler_kwargs: dict | None = None):
        self.optim = optim
        self.model = model
        self.max_norm = max_norm
        self.tp_group, self.pp_group = tp_group, pp_group
        self.expert_group = None  # set when experts are sharded over a group: their share of the norm is summed over it
        self.scaler = DynamicLossScaler(**(scaler_kwargs or {})) if precision == "fp16" else None
        if isinstance(optim, FusedAdamW):
            optim.max_norm = max_norm
            optim.norm_groups = [g for g in (tp_group, pp_group) if g is not None]

    @property
    def param_groups(self):
        return self.optim.param_groups

    def backward(self, loss: torch.Tensor, **kw):
        if self.scaler is not None:
            loss = loss * self.scaler.scale
        loss.backward(**kw)

    def backward_by_grad(self, tensors, grads):
        if self.scaler is not None:
            grads = [g * self.scaler.scale for g in grads]
        torch.autograd.backward(tensors, grads)

    def clip_grad_norm(self, max_norm: float | None = None) -> torch.Tensor | None:
        """Plain-optimizer path: clip ``.grad`` by the global norm over tp / pp groups (FusedAdamW clips inside its step)."""
        max_norm = self.max_norm if max_norm is None else max_norm
        if isinstance(self.optim, FusedAdamW) or max_norm <= 0:
            return None
        params = [p for g in self.optim.param_groups for p in g["params"] if p.grad is not None]
        if not params:
            return None
        sq = torch.zeros((), dtype=torch.float32, device=params[0].device)
        sq_expert = torch.zeros_like(sq)
        for p in params:
            # parameters replicated inside a tp group are counted once per rank; divide their share
            if getattr(p, "expert_parallel", False):
                sq_expert = sq_expert + p.grad.float().pow(2).sum()
            else:
                sq = sq + p.grad.float().pow(2).sum()
        if self.expert_group is not None and dist.get_world_size(self.expert_group) > 1:
            dist.all_reduce(sq_expert, group=self.expert_group)  # every rank owns different experts
        sq = sq + sq_expert
        for grp in (self.tp_group, self.pp_group):
            if grp is not None and dist.get_world_size(grp) > 1:
                dist.all_reduce(sq, group=grp)
        norm = sq.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
        for p in params:
            p.grad.mul_(coef.to(p.grad.dtype))
        return norm

    def step(self, *a, **kw):
        if self.scaler is not None:
            inv = 1.0 / self.scaler.scale
            if isinstance(self.optim, FusedAdamW):
                self.optim.loss_scale = self.scaler.scale
            else:
                overflow = False
                for g in self.optim.param_groups:
                    for p in g["params"]:
                        if p.grad is not None:
                            p.grad.mul_(inv)
                            overflow |= not bool(torch.isfinite(p.grad).all())
                self.scaler.update(overflow)
                if overflow:
                    self.optim.zero_grad()
                    return None
        self.clip_grad_norm()
        return self.optim.step(*a, **kw)

    def zero_grad(self, *a, **kw):
        return self.optim.zero_grad(*a, **kw)

    def state_dict(self):
        return self.optim.state_dict()

    def load_state_dict(self, sd):
        return self.optim.load_state_dict(sd)

    def update_master_params(self, model=None):
        if hasattr(self.optim, "update_master_params"):
            self.optim.update_master_params()

    def unwrap(self):
        return self.optim


class HybridParallelNaiveOptimizer(OptimizerWrapper):
    """The wrapper under the name the reference's plugin uses for fp32 / bf16 training."""

    def __init__(self, optim, model=None, max_norm: float = 0.0, tp_group=None, pp_group=None, **kw):
        super().__init__(optim, model, max_norm, None, tp_group, pp_group)


class HybridParallelAMPOptimizer(OptimizerWrapper):
    """The wrapper under the name the reference's plugin uses for mixed precision: ``precision="fp16"`` turns the dynamic
    loss scale on (``initial_scale``, ``min_scale``, ``growth_factor``, ``backoff_factor``, ``growth_interval``,
    ``hysteresis``, ``max_scale`` as in the reference's constructor)."""

    def __init__(self, optim, model=None, precision: str = "fp16", max_norm: float = 0.0, tp_group=None, pp_group=None,
                 **scaler_kwargs):
        super().__init__(optim, model, max_norm, precision, tp_group, pp_group, scaler_kwargs or None)
