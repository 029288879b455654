"""Fully-sharded data parallelism for a :class:`MultimodalModel` through PyTorch's FSDP2 (``fully_shard``).

The reference does not implement FSDP itself either: its example wraps every element of every ``ModuleList`` (the
transformer layers of each encoder and of the language model) and then the root
(examples/distributed/run_vlm_fsdp.py:133-139, docs/parallelization/ddp_fsdp.md).  ``shard_fully`` does the same walk.
During forward and backward FSDP2 hands the layers ordinary (all-gathered) tensors, so the kernels of this package see
what they see without it; parameters are sharded ``DTensor`` s in between, which is why the optimizer has to be a
PyTorch optimizer (``torch.optim.AdamW(model.parameters(), fused=True)``) and not the flat-arena ``FusedAdamW``.
``FusedAdamW(zero_stage=1)`` is the in-house alternative that shards only optimizer state.
"""

from __future__ import annotations

import torch.nn as nn


def shard_fully(model: nn.Module, mesh=None, reshard_after_forward: bool | None = None, mp_policy=None) -> nn.Module:
    """Apply ``fully_shard`` to every transformer layer (each element of each ``ModuleList``) and to ``model`` itself."""
    from torch.distributed.fsdp import fully_shard

    # None keeps FSDP2's own choice: layers free their gathered weights after forward, the root (embeddings, final norm,
    # head: needed again at the start of backward) keeps them
    kw = {} if reshard_after_forward is None else dict(reshard_after_forward=reshard_after_forward)
    if mesh is not None:
        kw["mesh"] = mesh
    if mp_policy is not None:
        kw["mp_policy"] = mp_policy
    for module in list(model.modules()):
        if isinstance(module, nn.ModuleList):
            for layer in module:
                if any(p.requires_grad for p in layer.parameters()):
                    fully_shard(layer, **kw)
    # projectors recompute their forward in the backward pass (gradient checkpointing): as units of their own they are
    # gathered again when that forward runs, which parameters left to the root unit are not
    from ..multimodal.modeling import MultimodalProjector

    for module in list(model.modules()):
        if isinstance(module, MultimodalProjector) and any(p.requires_grad for p in module.parameters()):
            fully_shard(module.projection, **kw)  # the inner module returns a plain tensor, which FSDP2 can hook
    fully_shard(model, **kw)
    return model
