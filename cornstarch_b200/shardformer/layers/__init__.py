"""Layer names as scripts written for the reference know them.

The reference takes its tensor-parallel layers from ColossalAI (``Linear1D_Col``, ``Linear1D_Row``,
``FusedLinear1D_Col``, ``VocabParallelEmbedding1D``, ``VocabParallelLMHead1D``, ``PaddingEmbedding``, ``PaddingLMHead``,
``FusedRMSNorm``, ``FusedLayerNorm``, ``DropoutForReplicatedInput``; cornstarch/shardformer/policies/llama.py:7-15,
cornstarch/shardformer/policies/siglip.py:6-10, cornstarch/shardformer/policies/phi3.py, cornstarch/shardformer/policies/dinov2.py:131).
Here they are the layers of :mod:`cornstarch_b200.nn`, which run this package's kernels; every one has
``from_native_module(module, process_group, **kwargs)``.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from ... import nn as cnn

Linear1D_Col = cnn.ColumnParallelLinear
Linear1D_Row = cnn.RowParallelLinear
VocabParallelEmbedding1D = cnn.VocabParallelEmbedding
DropoutForReplicatedInput = cnn.DropoutForReplicatedInput


class FusedLinear1D_Col(cnn.ColumnParallelLinear):
    """Column-parallel linear whose output is several projections side by side (``qkv_proj``, ``gate_up_proj``):
    ``split_sizes`` gives the width of each part, and every part is sharded on its own."""

    @classmethod
    def from_native_module(cls, module, process_group, split_sizes: list[int] | None = None, gather_output: bool = False, **kw):
        assert split_sizes, "FusedLinear1D_Col needs split_sizes"
        return super().from_native_module(module, process_group, gather_output=gather_output, split_sizes=list(split_sizes))


class PaddingEmbedding(cnn.VocabParallelEmbedding):
    """Embedding whose vocabulary is padded to a multiple of ``make_vocab_size_divisible_by`` without being sharded
    (what the reference uses when tensor parallelism is off): a vocab-parallel embedding over a group of one."""

    @classmethod
    def from_native_module(cls, module, process_group=None, make_vocab_size_divisible_by: int = 64, **kw):
        return super().from_native_module(module, None, divisible_by=make_vocab_size_divisible_by)


class VocabParallelLMHead1D(cnn.ColumnParallelLinear):
    """LM head sharded over the vocabulary, rows padded to a multiple of ``make_vocab_size_divisible_by * tp``."""

    @classmethod
    def from_native_module(cls, module, process_group, make_vocab_size_divisible_by: int = 64, gather_output: bool = False, **kw):
        tp = cnn._ws(process_group)
        V, H = module.weight.shape
        mult = make_vocab_size_divisible_by * tp
        Vp = (V + mult - 1) // mult * mult
        padded = cnn.Linear(H, Vp, bias=module.bias is not None, device=module.weight.device, dtype=module.weight.dtype)
        with torch.no_grad():
            padded.weight.zero_()
            padded.weight[:V].copy_(module.weight)
            if module.bias is not None:
                padded.bias.zero_()
                padded.bias[:V].copy_(module.bias)
        new = super().from_native_module(padded, process_group, gather_output=gather_output)
        new.num_embeddings = V
        return new


class PaddingLMHead(VocabParallelLMHead1D):
    """Padded but not sharded LM head (tensor parallelism off)."""

    @classmethod
    def from_native_module(cls, module, process_group=None, make_vocab_size_divisible_by: int = 64, **kw):
        return super().from_native_module(module, None, make_vocab_size_divisible_by=make_vocab_size_divisible_by)


class FusedRMSNorm(cnn.RMSNorm):
    @classmethod
    def from_native_module(cls, module, *args, **kw):
        eps = getattr(module, "eps", None) or getattr(module, "variance_epsilon", 1e-6)
        new = cls(module.weight.shape[0], eps, getattr(module, "weight_offset", 0.0), device=module.weight.device,
                  dtype=module.weight.dtype)
        new.weight = module.weight
        return new


class FusedLayerNorm(cnn.LayerNorm):
    @classmethod
    def from_native_module(cls, module, *args, **kw):
        new = cls(module.weight.shape[0], module.eps, device=module.weight.device, dtype=module.weight.dtype)
        new.weight = module.weight
        if getattr(module, "bias", None) is not None:
            new.bias = module.bias
        return new


class LazyInitContext:
    """Build a model without allocating its parameters (``with LazyInitContext(): model = Model(config)``), then give
    storage only to what a rank keeps: ``ShardFormer.optimize`` materialises the held layers, and
    ``LazyInitContext.materialize(module)`` does it for a whole module.  Stands in for ColossalAI's class of the same
    name used by the reference's tests (tests/test_shardformer/utils.py:16,317-329): construction on the meta device."""

    def __init__(self, default_device=None):
        self._ctx = torch.device("meta")
        self.default_device = default_device

    def __enter__(self):
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)

    @staticmethod
    def materialize(module: nn.Module, device=None, dtype=None) -> nn.Module:
        from ..shard.shardformer import materialize_meta

        materialize_meta(module, device, dtype)
        return module


__all__ = ["Linear1D_Col", "Linear1D_Row", "FusedLinear1D_Col", "VocabParallelEmbedding1D", "VocabParallelLMHead1D",
           "PaddingEmbedding", "PaddingLMHead", "FusedRMSNorm", "FusedLayerNorm", "DropoutForReplicatedInput",
           "LazyInitContext"]
