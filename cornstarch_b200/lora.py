"""Low-rank adapters on this package's linear layers (what the reference gets from ``peft`` in
examples/pretrain_vlm_lora.py:58-83): ``W x + (alpha / r) * B (A x)`` with the base weight frozen.

    from cornstarch_b200.lora import add_lora, merge_lora
    add_lora(model.language_model, r=16, alpha=32, target=("q_proj", "v_proj"))
    ...train...
    merge_lora(model.language_model)          # fold the adapters into the base weights

Both adapter GEMMs run on the same kernels as every other linear layer.  Layers that are fused with neighbours
(q|k|v or gate|up in one GEMM) keep that fusion for the base path; the call site adds ``delta(x)`` to the adapted
projection's slice of the fused output (``ops.linear.add_adapter_deltas``).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from . import nn as cnn
from .ops.linear import linear


class LoRALinear(nn.Module):
    def __init__(self, base: cnn.Linear, r: int, alpha: float, dropout: float = 0.0):
        super().__init__()
        self.base = base
        self.r, self.scaling = r, alpha / r
        dev, dt = base.weight.device, base.weight.dtype
        self.lora_A = nn.Parameter(torch.empty(r, base.in_features, device=dev, dtype=dt))
        self.lora_B = nn.Parameter(torch.zeros(base.out_features, r, device=dev, dtype=dt))
        nn.init.kaiming_uniform_(self.lora_A, a=math.sqrt(5))
        base.weight.requires_grad_(False)
        if base.bias is not None:
            base.bias.requires_grad_(False)
        self.drop = nn.Dropout(dropout) if dropout else None

    # the attributes fused call sites read
    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    @property
    def in_features(self):
        return self.base.in_features

    @property
    def out_features(self):
        return self.base.out_features

    def input_hook(self, x):
        return self.base.input_hook(x)

    def tp_spec(self, x):
        return None

    def delta(self, x):
        """The additive low-rank update (what fused call sites add to this projection's slice of their output)."""
        h = self.drop(x) if self.drop is not None else x
        return linear(linear(h, self.lora_A), self.lora_B) * self.scaling

    def forward(self, x):
        return self.base(x) + self.delta(x)

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight + (self.lora_B.float() @ self.lora_A.float()).to(self.base.weight.dtype) * self.scaling


def add_lora(model: nn.Module, r: int = 8, alpha: float = 16.0, target=("q_proj", "v_proj"), dropout: float = 0.0) -> list[str]:
    """Wrap every ``cnn.Linear`` whose attribute name is in ``target``; returns the wrapped module paths."""
    done = []
    for path, mod in list(model.named_modules()):
        for name, child in list(mod.named_children()):
            if name in target and isinstance(child, cnn.Linear) and not isinstance(child, LoRALinear):
                setattr(mod, name, LoRALinear(child, r, alpha, dropout))
                done.append(f"{path}.{name}" if path else name)
    return done


def merge_lora(model: nn.Module) -> None:
    for mod in list(model.modules()):
        for name, child in list(mod.named_children()):
            if isinstance(child, LoRALinear):
                with torch.no_grad():
                    child.base.weight.copy_(child.merged_weight())
                setattr(mod, name, child.base)
