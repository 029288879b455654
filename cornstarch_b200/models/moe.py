"""Mixture-of-experts decoder blocks (Mixtral, Qwen3-MoE) with an expert-parallel path.

Single-device semantics follow the HF blocks the reference keeps
(cornstarch/shardformer/modeling/mixtral.py: softmax over experts, top-k, renormalise, weighted sum of
SwiGLU experts; auxiliary load-balancing loss :419-430).  Tokens are sorted by expert once and each
expert runs three tcgen05 GEMMs over its contiguous token segment (a grouped GEMM as a loop over ragged
segments).  With an expert-parallel group (``ep_group``) every rank owns ``num_experts / ep`` experts and
tokens travel through :mod:`cornstarch_b200.parallel.ep` (dispatch / combine all-to-all), a capability
the reference does not have (its experts are only tensor-parallel,
cornstarch/shardformer/policies/mixtral.py:216-234).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import nn as cnn
from ..ops import elementwise as E
from ..ops.linear import multi_linear
from .base import register_model
from .llama import DecoderConfig, DecoderForCausalLM


class MixtralConfig(DecoderConfig):
    model_type = "mixtral"

    def __init__(self, num_local_experts=8, num_experts_per_tok=2, router_aux_loss_coef=0.001, output_router_logits=False,
                 **kw):
        self.num_local_experts = num_local_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.router_aux_loss_coef = router_aux_loss_coef
        self.output_router_logits = output_router_logits
        kw.setdefault("intermediate_size", 14336)
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("rope_theta", 1e6)
        super().__init__(**kw)


class Qwen3MoeConfig(DecoderConfig):
    model_type = "qwen3_moe"

    def __init__(self, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=768, norm_topk_prob=True,
                 decoder_sparse_step=1, mlp_only_layers=None, router_aux_loss_coef=0.001, num_local_experts=None, **kw):
        if num_local_experts is not None:
            num_experts = num_local_experts  # the name newer ``transformers`` releases write into config.json
        self.num_experts = self.num_local_experts = num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.moe_intermediate_size = moe_intermediate_size
        self.norm_topk_prob = norm_topk_prob
        self.decoder_sparse_step = decoder_sparse_step
        self.mlp_only_layers = mlp_only_layers or []
        self.router_aux_loss_coef = router_aux_loss_coef
        super().__init__(**kw)


class _SwiGLUExpert(nn.Module):
    """Mixtral names: w1 = gate, w3 = up, w2 = down."""

    def __init__(self, hidden, inter, names=("w1", "w3", "w2")):
        super().__init__()
        self.names = names
        setattr(self, names[0], cnn.Linear(hidden, inter, bias=False))
        setattr(self, names[1], cnn.Linear(hidden, inter, bias=False))
        setattr(self, names[2], cnn.Linear(inter, hidden, bias=False))

    def forward(self, x, act="silu"):
        g, u, d = (getattr(self, n) for n in self.names)
        gu = multi_linear(g.input_hook(x), [g.weight, u.weight], tp=g.tp_spec(x))
        return d(E.glu(gu, act))


def experts_forward_grouped(experts, x3: torch.Tensor, act: str) -> torch.Tensor:
    """``experts[e](x3[e])`` for every local expert, ``x3`` being ``[experts, rows, hidden]`` with the same number of rows
    for each: the gate / up projections of all experts run as one grouped GEMM, the GLU once over all rows, the down
    projections as one grouped GEMM (``ops.linear.grouped_multi_linear``).  Experts whose linears are wrapped or
    tensor-parallel run one after the other."""
    L, R, H = x3.shape
    if L == 1 or not all(type(getattr(e, n)) is cnn.Linear for e in experts for n in e.names):
        return torch.stack([experts[e](x3[e], act) for e in range(L)], dim=0)
    from ..ops.linear import grouped_multi_linear

    gate_up = [[getattr(e, e.names[0]).weight, getattr(e, e.names[1]).weight] for e in experts]
    down = [[getattr(e, e.names[2]).weight] for e in experts]
    gu = grouped_multi_linear(x3.reshape(L * R, H), gate_up, R)
    return grouped_multi_linear(E.glu(gu, act), down, R).view(L, R, H)


def route_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """softmax over experts -> top-k -> (optionally) renormalise.  Returns ``(weights [T,k], experts [T,k])``."""
    probs = F.softmax(router_logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, idx


def moe_forward_local(x2: torch.Tensor, weights, experts_idx, experts: nn.ModuleList, act: str, expert_offset: int = 0):
    """Run tokens through the experts held locally: sort by expert, one SwiGLU per contiguous segment, weighted scatter back."""
    T, H = x2.shape
    k = experts_idx.shape[1]
    flat_e = experts_idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    token_of = torch.div(order, k, rounding_mode="floor")
    sorted_e = flat_e[order]
    n_local = len(experts)
    counts = torch.bincount((sorted_e - expert_offset).clamp(0, n_local - 1), minlength=n_local)
    xin = x2[token_of]
    outs = []
    start = 0
    counts_host = counts.tolist()
    for e, n in enumerate(counts_host):
        seg = xin[start : start + n]
        outs.append(experts[e](seg, act) if n > 0 else seg.new_zeros((0, H)))
        start += n
    y = torch.cat(outs, dim=0)
    y = y * weights.reshape(-1)[order].unsqueeze(-1).to(y.dtype)
    out = torch.zeros_like(x2)
    out.index_add_(0, token_of, y)
    return out


class MixtralSparseMoeBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.top_k = config.num_experts_per_tok
        self.num_experts = config.num_local_experts
        self.act = config.hidden_act
        self.gate = cnn.Linear(config.hidden_size, self.num_experts, bias=False)
        self.experts = nn.ModuleList(
            [_SwiGLUExpert(config.hidden_size, config.intermediate_size) for _ in range(self.num_experts)])
        self.ep = None  # cornstarch_b200.parallel.ep.ExpertParallel when experts are sharded across ranks
        self.renormalize = True

    def forward(self, x):
        B, S, H = x.shape
        x2 = x.reshape(-1, H)
        logits = self.gate(x2)
        w, idx = route_topk(logits, self.top_k, self.renormalize)
        if self.ep is not None:
            out = self.ep.forward(x2, w, idx, self.experts, self.act)
        else:
            out = moe_forward_local(x2, w, idx, self.experts, self.act)
        return out.view(B, S, H), logits


class Qwen3MoeSparseMoeBlock(MixtralSparseMoeBlock):
    def __init__(self, config):
        nn.Module.__init__(self)
        self.top_k = config.num_experts_per_tok
        self.num_experts = config.num_experts
        self.act = config.hidden_act
        self.gate = cnn.Linear(config.hidden_size, self.num_experts, bias=False)
        self.experts = nn.ModuleList([
            _SwiGLUExpert(config.hidden_size, config.moe_intermediate_size, ("gate_proj", "up_proj", "down_proj"))
            for _ in range(self.num_experts)])
        self.ep = None
        self.renormalize = bool(config.norm_topk_prob)


def load_balancing_loss(router_logits, num_experts: int, top_k: int, attention_mask=None) -> torch.Tensor:
    """Switch-transformer auxiliary loss over all layers: ``E * sum_e f_e * P_e`` (HF ``load_balancing_loss_func``)."""
    if not router_logits:
        return torch.zeros(())
    logits = torch.cat([r.reshape(-1, num_experts) for r in router_logits], dim=0).float()
    probs = F.softmax(logits, dim=-1)
    _, sel = torch.topk(probs, top_k, dim=-1)
    onehot = F.one_hot(sel, num_experts).float()  # [N, k, E]
    if attention_mask is None:
        tokens_per_expert = onehot.mean(dim=0)  # [k, E]
        prob_per_expert = probs.mean(dim=0)
    else:
        L = len(router_logits)
        m = attention_mask.reshape(-1).float().repeat(L)
        tokens_per_expert = (onehot * m[:, None, None]).sum(0) / m.sum().clamp(min=1)
        prob_per_expert = (probs * m[:, None]).sum(0) / m.sum().clamp(min=1)
    return (tokens_per_expert * prob_per_expert.unsqueeze(0)).sum() * num_experts


class MoeForCausalLM(DecoderForCausalLM):
    """Mixtral / Qwen3-MoE causal LM: adds the router auxiliary loss to the LM loss."""

    def forward(self, *args, output_router_logits: bool | None = None, **kwargs):
        out = super().forward(*args, **kwargs)
        cfg = self.config
        coef = getattr(cfg, "router_aux_loss_coef", 0.0)
        want = output_router_logits if output_router_logits is not None else getattr(cfg, "output_router_logits", False)
        if want and out.get("router_logits") and "loss" in out and coef:
            E_ = getattr(cfg, "num_local_experts", None) or getattr(cfg, "num_experts")
            aux = load_balancing_loss(out["router_logits"], E_, cfg.num_experts_per_tok)
            out["aux_loss"] = aux
            out["loss"] = out["loss"] + coef * aux.to(out["loss"].dtype)
        return out


MixtralForCausalLM = MoeForCausalLM
register_model("mixtral", MixtralConfig, MoeForCausalLM)
register_model("qwen3_moe", Qwen3MoeConfig, MoeForCausalLM)
