"""Building-block modules: linears (plain / column- / row-parallel), embeddings, norms.

All of them keep HF-compatible parameter names (``weight``, ``bias``) and route their math through
:mod:`cornstarch_b200.ops` (native sm_100a kernels for bf16 CUDA tensors, PyTorch otherwise).

The tensor-parallel classes are this framework's ``Linear1D_Col`` / ``Linear1D_Row`` /
``VocabParallelEmbedding1D`` / ``VocabParallelLMHead1D`` (imported from ColossalAI by the reference,
cornstarch/shardformer/policies/llama.py:7-15): ``from_native_module(module, process_group)`` slices
an existing module's parameters for this rank.  Activations are replicated across the TP group
(column-parallel: identity forward / all-reduce backward on the input; row-parallel: all-reduce forward
on the output), matching the reference's Megatron-1D layout.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .ops import _native as nat

from .ops import elementwise as E
from .ops.linear import linear, multi_linear
from .parallel import comm


def _ws(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _rank(group) -> int:
    return 0 if group is None else dist.get_rank(group)


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type == "meta":
            return
        nn.init.normal_(self.weight, std=0.02)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x):
        return linear(x, self.weight, self.bias)

    # hooks used by callers that fuse several projections into one GEMM and therefore bypass forward()
    def input_hook(self, x):
        return x

    def tp_spec(self, x):
        """``("col" | "row", FusedTensorParallel)`` when the tensor-parallel reduce can be fused into the GEMM."""
        return None

    def output_hook(self, y):
        return y

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


class ColumnParallelLinear(Linear):
    """Output features sharded over the TP group: ``weight`` is ``[out/tp, in]``."""

    def __init__(self, in_features, out_features, bias=True, process_group=None, gather_output=False, device=None,
                 dtype=None):
        self.process_group = process_group
        self.gather_output = gather_output
        self.full_out_features = out_features
        tp = _ws(process_group)
        assert out_features % tp == 0, f"out_features {out_features} not divisible by tp {tp}"
        super().__init__(in_features, out_features // tp, bias, device, dtype)

    @classmethod
    def from_native_module(cls, module: Linear, process_group, gather_output: bool = False, n_fused: int = 1,
                           split_sizes: list[int] | None = None):
        """Slice ``module``; ``split_sizes`` handles fused projections (qkv / gate_up) whose parts are sharded separately."""
        tp, r = _ws(process_group), _rank(process_group)
        w, b = module.weight.data, (module.bias.data if module.bias is not None else None)
        new = cls(module.in_features, module.out_features, b is not None, process_group, gather_output, device="meta",
                  dtype=w.dtype)
        new.weight = nn.Parameter(shard_rows(w, tp, r, split_sizes).clone(), requires_grad=module.weight.requires_grad)
        if b is not None:
            new.bias = nn.Parameter(shard_rows(b, tp, r, split_sizes).clone(), requires_grad=module.bias.requires_grad)
        new.split_sizes = split_sizes
        return new

    def tp_spec(self, x):
        ftp = _fused_tp(self.process_group, x)
        return ("col", ftp) if ftp is not None else None

    def input_hook(self, x):
        if self.tp_spec(x) is not None:
            return x  # the backward all-reduce of dx happens inside the fused GEMM
        return comm.reduce_backward(x, self.process_group)

    def forward(self, x):
        spec = self.tp_spec(x)
        if spec is None:
            x = comm.reduce_backward(x, self.process_group)
        y = linear(x, self.weight, self.bias, tp=spec)
        if self.gather_output:
            y = comm.gather_forward_split_backward(y, -1 % y.dim(), self.process_group)
        return y


class RowParallelLinear(Linear):
    """Input features sharded over the TP group: ``weight`` is ``[out, in/tp]``; the bias is added after the reduce."""

    def __init__(self, in_features, out_features, bias=True, process_group=None, device=None, dtype=None):
        self.process_group = process_group
        self.full_in_features = in_features
        tp = _ws(process_group)
        assert in_features % tp == 0, f"in_features {in_features} not divisible by tp {tp}"
        super().__init__(in_features // tp, out_features, bias, device, dtype)

    @classmethod
    def from_native_module(cls, module: Linear, process_group, split_sizes: list[int] | None = None):
        tp, r = _ws(process_group), _rank(process_group)
        w = module.weight.data
        new = cls(module.in_features, module.out_features, module.bias is not None, process_group, device="meta",
                  dtype=w.dtype)
        new.weight = nn.Parameter(shard_rows(w.t(), tp, r, split_sizes).t().contiguous(),
                                  requires_grad=module.weight.requires_grad)
        if module.bias is not None:
            new.bias = nn.Parameter(module.bias.data.clone(), requires_grad=module.bias.requires_grad)
        return new

    def output_hook(self, y):
        y = comm.reduce_forward(y, self.process_group)
        if self.bias is not None:
            y = y + self.bias
        return y

    def tp_spec(self, x):
        ftp = _fused_tp(self.process_group, x)
        return ("row", ftp) if ftp is not None else None

    def forward(self, x):
        spec = self.tp_spec(x)
        if spec is not None:
            y = linear(x, self.weight, None, tp=spec)
            return y + self.bias if self.bias is not None else y
        return self.output_hook(linear(x, self.weight, None))


FUSED_TP_ENABLED = True


def _fused_tp(group, x):
    """The fused GEMM + all-reduce context of ``group`` for bf16 CUDA inputs (``None`` = use NCCL collectives)."""
    if not FUSED_TP_ENABLED or nat.LIBRARY_MODE or group is None or not x.is_cuda or x.dtype != torch.bfloat16:
        return None
    from .parallel.symm import FusedTensorParallel

    return FusedTensorParallel.get(group)


def shard_rows(t: torch.Tensor, tp: int, rank: int, split_sizes: list[int] | None = None) -> torch.Tensor:
    """Rank's slice of dim 0; with ``split_sizes`` every fused part is sliced separately and re-concatenated."""
    if tp == 1:
        return t
    if not split_sizes:
        return t.chunk(tp, dim=0)[rank]
    parts = torch.split(t, split_sizes, dim=0)
    return torch.cat([p.chunk(tp, dim=0)[rank] for p in parts], dim=0)


def unshard_rows(shards: list[torch.Tensor], split_sizes: list[int] | None = None) -> torch.Tensor:
    """Inverse of :func:`shard_rows` given every rank's slice (checkpoint save gathers with this)."""
    tp = len(shards)
    if tp == 1:
        return shards[0]
    if not split_sizes:
        return torch.cat(shards, dim=0)
    local = [s // tp for s in split_sizes]
    per_rank = [torch.split(s, local, dim=0) for s in shards]
    return torch.cat([torch.cat([per_rank[r][i] for r in range(tp)], dim=0) for i in range(len(split_sizes))], dim=0)


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, padding_idx=None, device=None, dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim, self.padding_idx = num_embeddings, embedding_dim, padding_idx
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device, dtype=dtype))
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids: torch.Tensor, feats: torch.Tensor | None = None, src: torch.Tensor | None = None):
        """Plain lookup, or (``src`` given) lookup fused with the scatter of encoder features."""
        if src is not None:
            out = E.embed_merge(self.weight, src.reshape(-1), feats)
            return out.view(*ids.shape, self.embedding_dim)
        if self.weight.is_cuda and self.weight.dtype == torch.bfloat16 and not nat.LIBRARY_MODE:
            out = E.embed_merge(self.weight, ids.reshape(-1).int(), None)
            return out.view(*ids.shape, self.embedding_dim)
        return F.embedding(ids, self.weight)


class VocabParallelEmbedding(Embedding):
    """Vocabulary rows sharded over the TP group (vocab padded to a multiple of ``divisible_by * tp``)."""

    def __init__(self, num_embeddings, embedding_dim, process_group=None, divisible_by: int = 64, device=None,
                 dtype=None):
        tp = _ws(process_group)
        mult = divisible_by * tp
        self.full_num_embeddings = num_embeddings
        self.padded_num_embeddings = (num_embeddings + mult - 1) // mult * mult
        self.process_group = process_group
        local = self.padded_num_embeddings // tp
        super().__init__(local, embedding_dim, None, device, dtype)
        self.vocab_start = _rank(process_group) * local
        self.vocab_end = self.vocab_start + local

    @classmethod
    def from_native_module(cls, module: Embedding, process_group, divisible_by: int = 64):
        w = module.weight.data
        new = cls(module.num_embeddings, module.embedding_dim, process_group, divisible_by, device="meta", dtype=w.dtype)
        full = w
        if new.padded_num_embeddings != w.shape[0]:
            full = torch.cat([w, w.new_zeros(new.padded_num_embeddings - w.shape[0], w.shape[1])], dim=0)
        new.weight = nn.Parameter(full[new.vocab_start : new.vocab_end].clone(), requires_grad=module.weight.requires_grad)
        return new

    def forward(self, ids, feats=None, src=None):
        if _ws(self.process_group) == 1:
            return super().forward(ids, feats, src)
        assert src is None, "modality merge happens after the vocab-parallel reduce"
        inside = (ids >= self.vocab_start) & (ids < self.vocab_end)
        # Tokens of other ranks' shards look up SOME local row and are zeroed below.  They are spread over the rows
        # (modulo) instead of clamped onto the first / last one: thousands of tokens on one row made the embedding's
        # backward pass (a segmented sum per row) take about 10 ms per 8192-token micro-batch on the first pipeline stage.
        local = torch.remainder(ids - self.vocab_start, self.num_embeddings)
        out = F.embedding(local, self.weight)
        out = out * inside.unsqueeze(-1).to(out.dtype)
        return comm.reduce_forward(out, self.process_group)


class RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, weight_offset: float = 0.0, device=None, dtype=None):
        super().__init__()
        self.eps, self.weight_offset = eps, weight_offset
        init = torch.zeros if weight_offset else torch.ones
        self.weight = nn.Parameter(init(hidden_size, device=device, dtype=dtype))
        # A norm over the head dimension applied to the heads of ONE tensor-parallel rank (q_norm / k_norm) sees only
        # part of the heads: its weight gradient is the sum over the group.  The owner sets the group.
        self.grad_sum_group = None

    def forward(self, x, residual=None):
        w = self.weight
        if self.grad_sum_group is not None:
            w = comm.reduce_backward(w, self.grad_sum_group)  # identity forward, all-reduce of the gradient
        return E.rms_norm(x, w, self.eps, residual, self.weight_offset)


class LayerNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-5, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(hidden_size, device=device, dtype=dtype)) if bias else None

    def forward(self, x, residual=None):
        return E.layer_norm(x, self.weight, self.bias, self.eps, residual)


class DropoutForReplicatedInput(nn.Dropout):
    """Dropout whose mask is identical on every rank of a TP group (the input is replicated there)."""

    def __init__(self, p: float = 0.0, process_group=None):
        super().__init__(p)
        self.process_group = process_group

    def forward(self, x):
        if not self.training or self.p == 0.0:
            return x
        seed = torch.randint(0, 2**31 - 1, (1,), device=x.device)
        if _ws(self.process_group) > 1:
            dist.broadcast(seed, src=dist.get_global_rank(self.process_group, 0), group=self.process_group)
        g = torch.Generator(device=x.device).manual_seed(int(seed.item()))
        keep = torch.rand(x.shape, generator=g, device=x.device) >= self.p
        return x * keep.to(x.dtype) / (1.0 - self.p)


def qkv_linear(x, q: Linear, k: Linear, v: Linear):
    """The three attention projections as one GEMM when their weights are adjacent in memory."""
    return multi_linear(x, [q.weight, k.weight, v.weight], [q.bias, k.bias, v.bias] if q.bias is not None or v.bias is not None else None,
                        tp=q.tp_spec(x))


def init_std(hidden: int) -> float:
    return 1.0 / math.sqrt(hidden)
