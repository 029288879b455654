"""``TensorPlaceholder``: what is left of a parameter after its storage was released.

A stage that does not hold a layer keeps only this record (id, shape, dtype, requires_grad), so the
model can be re-sharded later (a re-plan after a membership change) and the tensor re-created with
``create``.  Same role as cornstarch/shardformer/shard/placeholder.py:5-29 in the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class TensorPlaceholder:
    param_id: int
    shape: torch.Size
    dtype: torch.dtype
    requires_grad: bool

    def __init__(self, input_tensor: torch.Tensor):
        self.param_id = id(input_tensor)
        self.shape = input_tensor.shape
        self.dtype = input_tensor.dtype
        self.requires_grad = input_tensor.requires_grad

    def create(self, device=None, dtype=None) -> torch.Tensor:
        t = torch.empty(self.shape, dtype=dtype or self.dtype, device=device)
        return torch.nn.Parameter(t, requires_grad=self.requires_grad) if self.requires_grad else t
