"""Decoder-only LLM family (Llama, Mistral, Qwen2, Qwen3, Gemma, Gemma2, Gemma3-text, Phi3) on fused kernels.

One implementation, configured by ``model_type``-specific flags (:func:`decoder_spec`), with HF parameter
names so HF checkpoints load unchanged.  Covers what the reference does with one policy + one patched
forward per family (cornstarch/shardformer/policies/{llama,mistral,qwen2,qwen3,gemma,gemma2,gemma3,phi3}.py and
cornstarch/shardformer/modeling/*): pipeline stages (only held layers run; non-last stages return
``hidden_states``), tensor parallelism (column/row-parallel projections, vocab-parallel embedding and
LM head with a fused vocab-parallel cross-entropy), context parallelism (token subsets with explicit
positions) and Ulysses sequence parallelism.

Kernel mapping per layer: fused residual-add + RMSNorm -> one q|k|v GEMM -> in-place RoPE -> bitfield
flash attention -> o_proj GEMM -> fused residual-add + RMSNorm -> one gate|up GEMM -> SwiGLU -> down GEMM.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
from ..utils.recompute import checkpoint_layer

from .. import nn as cnn
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.cross_entropy import linear_cross_entropy
from ..nn import _fused_tp
from ..ops.linear import add_adapter_deltas, ag_linear, linear, multi_linear, rs_linear
from ..parallel import comm
from ..parallel.dp_fused import layer_input as grad_sync_layer_input
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, is_released, register_model


class DecoderConfig(PretrainedConfig):
    model_type = "llama"
    composite_key = "text_config"

    def __init__(self, vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                 num_attention_heads=32, num_key_value_heads=None, head_dim=None, hidden_act="silu",
                 max_position_embeddings=8192, rms_norm_eps=1e-6, rope_theta=10000.0, rope_scaling=None,
                 attention_bias=False, mlp_bias=False, tie_word_embeddings=False, pad_token_id=None,
                 initializer_range=0.02, **kwargs):
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_hidden_layers = num_hidden_layers
        self.num_attention_heads = num_attention_heads
        self.num_key_value_heads = num_key_value_heads or num_attention_heads
        self.head_dim = head_dim or hidden_size // num_attention_heads
        self.hidden_act = hidden_act
        self.max_position_embeddings = max_position_embeddings
        self.rms_norm_eps = rms_norm_eps
        self.rope_theta = rope_theta
        self.rope_scaling = rope_scaling
        self.attention_bias = attention_bias
        self.mlp_bias = mlp_bias
        self.tie_word_embeddings = tie_word_embeddings
        self.pad_token_id = pad_token_id
        self.initializer_range = initializer_range
        super().__init__(**kwargs)


def _cfg_cls(mt: str, **defaults):
    def __init__(self, **kw):
        merged = dict(defaults)
        merged.update(kw)
        DecoderConfig.__init__(self, **merged)

    return type(f"{mt.title().replace('_', '')}Config", (DecoderConfig,), {"model_type": mt, "__init__": __init__})


LlamaConfig = DecoderConfig
MistralConfig = _cfg_cls("mistral")
Qwen2Config = _cfg_cls("qwen2", attention_bias=True)
Qwen3Config = _cfg_cls("qwen3")
GemmaConfig = _cfg_cls("gemma", hidden_act="gelu_pytorch_tanh", tie_word_embeddings=True)
Gemma2Config = _cfg_cls("gemma2", hidden_act="gelu_pytorch_tanh", tie_word_embeddings=True)
Gemma3TextConfig = _cfg_cls("gemma3_text", hidden_act="gelu_pytorch_tanh", tie_word_embeddings=True)
Phi3Config = _cfg_cls("phi3", rms_norm_eps=1e-5)


@dataclass
class DecoderSpec:
    """Per-family switches."""

    qkv_bias: bool = False
    o_bias: bool = False
    qk_norm: bool = False
    norm_offset: float = 0.0  # Gemma: weight stored as (w - 1)
    embed_scale: bool = False  # Gemma: embeddings * sqrt(hidden)
    sandwich_norm: bool = False  # Gemma2/3: post-attention and post-feedforward norms on the sub-layer output
    fused_names: bool = False  # Phi3: qkv_proj / gate_up_proj parameters
    local_rope: bool = False  # Gemma3: second rotary table for sliding layers
    attn_scale: float | None = None
    final_softcap: float | None = None
    moe: str | None = None  # "mixtral" | "qwen3_moe"


def decoder_spec(config) -> DecoderSpec:
    mt = getattr(config, "model_type", "llama")
    s = DecoderSpec()
    bias = bool(getattr(config, "attention_bias", False))
    s.qkv_bias, s.o_bias = bias, bias
    if mt == "qwen2":
        s.qkv_bias, s.o_bias = True, False
    elif mt in ("qwen3", "qwen3_moe"):
        s.qk_norm = True
        if mt == "qwen3_moe":
            s.moe = "qwen3_moe"
    elif mt == "gemma":
        s.norm_offset, s.embed_scale = 1.0, True
    elif mt in ("gemma2", "gemma3_text"):
        s.norm_offset, s.embed_scale, s.sandwich_norm = 1.0, True, True
        q = getattr(config, "query_pre_attn_scalar", None)
        s.attn_scale = (q ** -0.5) if q else None
        s.final_softcap = getattr(config, "final_logit_softcapping", None)
        if mt == "gemma3_text":
            s.qk_norm, s.local_rope = True, True
    elif mt == "phi3":
        s.fused_names = True
    elif mt == "mixtral":
        s.moe = "mixtral"
    return s


class ParallelContext:
    """Process groups a model shard works with (all optional)."""

    def __init__(self, tp_group=None, sp_group=None, sp_mode: str | None = None, cp_dist_mode=None, parallel_output=True,
                 tp_seq_shard: bool | None = None):
        self.tp_group = tp_group
        self.sp_group = sp_group
        self.sp_mode = sp_mode  # None | "ring_attn" | "all_to_all"
        self.cp_dist_mode = cp_dist_mode
        self.parallel_output = parallel_output
        if tp_seq_shard is None:
            import os

            tp_seq_shard = os.environ.get("CORNSTARCH_B200_TP_SEQ_SHARD", "0") == "1"
        # token-sharded activations between the tensor-parallel blocks (see ops/linear.py: ag_linear / rs_linear)
        self.tp_seq_shard = bool(tp_seq_shard)

    def seq_shard_group(self, tokens: int, hidden_like: torch.Tensor):
        """The tensor-parallel group when a ``tokens``-row activation can be token-sharded over it (whole 128-row tiles
        per rank on CUDA, an even split elsewhere), else ``None``: the layer then keeps replicated activations."""
        if not self.tp_seq_shard or self.tp_group is None or self.tp_size < 2 or (self.sp_mode and self.sp_size > 1):
            return None
        unit = 128 * self.tp_size if hidden_like.is_cuda else self.tp_size
        return self.tp_group if tokens % unit == 0 else None

    @property
    def tp_size(self):
        return comm._world(self.tp_group)

    @property
    def sp_size(self):
        return comm._world(self.sp_group)


class RotaryEmbedding(nn.Module):
    """Holds the fp32 cos/sin tables (non-persistent buffers); ``forward`` just returns them."""

    def __init__(self, config, theta: float | None = None, dim: int | None = None, scaling="config"):
        super().__init__()
        self.dim = dim or config.head_dim
        self.theta = theta if theta is not None else getattr(config, "rope_theta", 10000.0)
        self.max_pos = getattr(config, "max_position_embeddings", 8192)
        self.scaling = getattr(config, "rope_scaling", None) if scaling == "config" else scaling
        self._tables = None

    def tables(self, device, min_len: int = 0):
        need = max(self.max_pos, min_len)
        if self._tables is None or self._tables[0].device != torch.device(device) or self._tables[0].shape[0] < need:
            self._tables = E.rope_tables(need, self.dim, self.theta, device, self.scaling)
        return self._tables

    def forward(self, device, min_len: int = 0):
        return self.tables(device, min_len)


class Attention(nn.Module):
    def __init__(self, config, spec: DecoderSpec, layer_idx: int):
        super().__init__()
        self.config, self.spec, self.layer_idx = config, spec, layer_idx
        H, D = config.hidden_size, config.head_dim
        self.head_dim = D
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_key_value_heads
        self.scale = spec.attn_scale if spec.attn_scale is not None else 1.0 / math.sqrt(D)
        if spec.fused_names:
            self.qkv_proj = cnn.Linear(H, (self.num_heads + 2 * self.num_kv_heads) * D, bias=spec.qkv_bias)
        else:
            self.q_proj = cnn.Linear(H, self.num_heads * D, bias=spec.qkv_bias)
            self.k_proj = cnn.Linear(H, self.num_kv_heads * D, bias=spec.qkv_bias)
            self.v_proj = cnn.Linear(H, self.num_kv_heads * D, bias=spec.qkv_bias)
        self.o_proj = cnn.Linear(self.num_heads * D, H, bias=spec.o_bias)
        if spec.qk_norm:
            self.q_norm = cnn.RMSNorm(D, config.rms_norm_eps, spec.norm_offset)
            self.k_norm = cnn.RMSNorm(D, config.rms_norm_eps, spec.norm_offset)
        self.pc: ParallelContext | None = None
        self.attn_impl = None  # set by context parallelism

    def forward(self, x, rope, pos, mask: A.AttnMask, full_shape=None):
        """``full_shape = (B, S, group)``: ``x`` holds this rank's token rows of a ``[B, S]`` batch (token-sharded tensor
        parallelism); the q|k|v projection gathers the rows inside its GEMM, ``o_proj`` scatters them again."""
        B, S, _ = x.shape
        D, Hq, Hk = self.head_dim, self.num_heads, self.num_kv_heads
        sharded = full_shape is not None
        if sharded:
            B, S, tp_group = full_shape
            ws = [self.qkv_proj.weight] if self.spec.fused_names else [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight]
            qkv = ag_linear(x, ws, tp_group, _fused_tp(tp_group, x)).view(B, S, -1)
        elif self.spec.fused_names:
            qkv = self.qkv_proj(x)
        else:
            xin = self.q_proj.input_hook(x)
            biases = [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.spec.qkv_bias else None
            qkv = multi_linear(xin, [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight], biases, tp=self.q_proj.tp_spec(x))
            qkv = add_adapter_deltas(qkv, xin, (self.q_proj, self.k_proj, self.v_proj))
        ulysses = self.pc is not None and self.pc.sp_mode == "all_to_all" and self.pc.sp_size > 1
        if ulysses:
            # [B, S/sp, heads*D] -> [B, S, heads/sp*D] separately for q, k, v
            q, k, v = torch.split(qkv, [Hq * D, Hk * D, Hk * D], dim=-1)
            q, k, v = (comm.all_to_all_comm(t, self.pc.sp_group, 2, 1) for t in (q, k, v))
            sp = self.pc.sp_size
            Hq, Hk = Hq // sp, Hk // sp
            S = q.shape[1]
            qkv = torch.cat([q, k, v], dim=-1)
        if self.spec.qk_norm:
            q, k, v = torch.split(qkv, [Hq * D, Hk * D, Hk * D], dim=-1)
            q = self.q_norm(q.reshape(B, S, Hq, D)).reshape(B, S, Hq * D)
            k = self.k_norm(k.reshape(B, S, Hk, D)).reshape(B, S, Hk * D)
            qkv = torch.cat([q, k, v], dim=-1)
        if rope is not None:
            qkv = E.rope_(qkv, rope[0], rope[1], pos, Hq + Hk, D)
        q = qkv[..., : Hq * D].view(B, S, Hq, D)
        k = qkv[..., Hq * D : (Hq + Hk) * D].view(B, S, Hk, D)
        v = qkv[..., (Hq + Hk) * D :].view(B, S, Hk, D)
        if self.attn_impl is not None:
            o = self.attn_impl(q, k, v, mask, self.scale)
        else:
            o = A.attention(q, k, v, mask, self.scale)
        o = o.reshape(B, S, Hq * D)
        if ulysses:
            o = comm.all_to_all_comm(o, self.pc.sp_group, 1, 2)
        if sharded:
            return rs_linear(o, self.o_proj.weight, tp_group, _fused_tp(tp_group, o)).unsqueeze(0)
        return self.o_proj(o)


class MLP(nn.Module):
    def __init__(self, config, spec: DecoderSpec, intermediate_size: int | None = None):
        super().__init__()
        H, I = config.hidden_size, intermediate_size or config.intermediate_size
        bias = bool(getattr(config, "mlp_bias", False))
        self.act = config.hidden_act
        self.fused = spec.fused_names
        if self.fused:
            self.gate_up_proj = cnn.Linear(H, 2 * I, bias=bias)
        else:
            self.gate_proj = cnn.Linear(H, I, bias=bias)
            self.up_proj = cnn.Linear(H, I, bias=bias)
        self.down_proj = cnn.Linear(I, H, bias=bias)

    def forward(self, x, tp_group=None):
        if tp_group is not None:
            # token-sharded input: gather inside the gate|up GEMM, scatter inside the down GEMM
            ws = [self.gate_up_proj.weight] if self.fused else [self.gate_proj.weight, self.up_proj.weight]
            gu = ag_linear(x, ws, tp_group, _fused_tp(tp_group, x))
            return rs_linear(E.glu(gu, self.act), self.down_proj.weight, tp_group, _fused_tp(tp_group, gu)).unsqueeze(0)
        if self.fused:
            gu = self.gate_up_proj(x)
        else:
            xin = self.gate_proj.input_hook(x)
            biases = [self.gate_proj.bias, self.up_proj.bias] if self.gate_proj.bias is not None else None
            gu = multi_linear(xin, [self.gate_proj.weight, self.up_proj.weight], biases, tp=self.gate_proj.tp_spec(x))
            gu = add_adapter_deltas(gu, xin, (self.gate_proj, self.up_proj))
        return self.down_proj(E.glu(gu, self.act))


class DecoderLayer(nn.Module):
    def __init__(self, config, spec: DecoderSpec, layer_idx: int):
        super().__init__()
        self.spec = spec
        eps, off = config.rms_norm_eps, spec.norm_offset
        self.self_attn = Attention(config, spec, layer_idx)
        if spec.moe == "mixtral":
            from .moe import MixtralSparseMoeBlock

            self.block_sparse_moe = MixtralSparseMoeBlock(config)
        elif spec.moe == "qwen3_moe":
            from .moe import Qwen3MoeSparseMoeBlock

            sparse = (layer_idx not in getattr(config, "mlp_only_layers", [])) and (
                getattr(config, "num_experts", 0) > 0 and (layer_idx + 1) % getattr(config, "decoder_sparse_step", 1) == 0)
            self.mlp = Qwen3MoeSparseMoeBlock(config) if sparse else MLP(config, spec)
        else:
            self.mlp = MLP(config, spec)
        self.input_layernorm = cnn.RMSNorm(config.hidden_size, eps, off)
        self.post_attention_layernorm = cnn.RMSNorm(config.hidden_size, eps, off)
        if spec.sandwich_norm:
            self.pre_feedforward_layernorm = cnn.RMSNorm(config.hidden_size, eps, off)
            self.post_feedforward_layernorm = cnn.RMSNorm(config.hidden_size, eps, off)

    def _ffn(self, x, tp_group=None):
        if self.spec.moe == "mixtral":
            return self.block_sparse_moe(x)
        out = self.mlp(x, tp_group) if tp_group is not None else self.mlp(x)
        return out if isinstance(out, tuple) else (out, None)

    def supports_seq_shard(self) -> bool:
        """Token-sharded tensor parallelism covers dense blocks whose projections carry no bias."""
        a = self.self_attn
        if self.spec.moe or not isinstance(getattr(self, "mlp", None), MLP):
            return False
        lins = [a.o_proj, self.mlp.down_proj] + ([a.qkv_proj] if self.spec.fused_names else [a.q_proj, a.k_proj, a.v_proj])
        lins += [self.mlp.gate_up_proj] if self.mlp.fused else [self.mlp.gate_proj, self.mlp.up_proj]
        return all(l.bias is None and not hasattr(l, "delta") for l in lins)

    def forward(self, delta, residual, rope, pos, mask, full_shape=None):
        """``delta`` is the previous sub-layer output still to be added to the stream ``residual`` (None at a stage start).
        ``full_shape = (B, S, group)``: ``delta`` / ``residual`` hold this rank's token rows only (``[1, B*S/tp, H]``)."""
        if residual is None:
            residual = delta
            x = self.input_layernorm(delta)
        else:
            x, residual = self.input_layernorm(delta, residual)
        if full_shape is not None:
            a = self.self_attn(x, rope, pos, mask, full_shape)
            x, residual = self.post_attention_layernorm(a, residual)
            m, aux = self._ffn(x, full_shape[2])
            return m, residual, aux
        a = self.self_attn(x, rope, pos, mask)
        if self.spec.sandwich_norm:
            a = self.post_attention_layernorm(a)
            x, residual = self.pre_feedforward_layernorm(a, residual)
            m, aux = self._ffn(x)
            m = self.post_feedforward_layernorm(m)
        else:
            x, residual = self.post_attention_layernorm(a, residual)
            m, aux = self._ffn(x)
        return m, residual, aux


class DecoderModel(PreTrainedModel):
    """The ``LlamaModel``-shaped trunk: ``embed_tokens``, ``rotary_emb``, ``layers.N``, ``norm``."""

    config_class = DecoderConfig

    def __init__(self, config):
        super().__init__(config)
        self.spec = decoder_spec(config)
        self.embed_tokens = cnn.Embedding(config.vocab_size, config.hidden_size, getattr(config, "pad_token_id", None))
        self.layers = nn.ModuleList([DecoderLayer(config, self.spec, i) for i in range(config.num_hidden_layers)])
        self.norm = cnn.RMSNorm(config.hidden_size, config.rms_norm_eps, self.spec.norm_offset)
        self.rotary_emb = RotaryEmbedding(config)
        if self.spec.local_rope:
            self.rotary_emb_local = RotaryEmbedding(config, theta=getattr(config, "rope_local_base_freq", 10000.0), scaling=None)
        self.pc: ParallelContext | None = None
        self._init_weights()

    def _init_weights(self):
        std = getattr(self.config, "initializer_range", 0.02)
        for p in self.parameters():
            if p.device.type != "meta" and p.dim() >= 2:
                nn.init.normal_(p, std=std)

    @classmethod
    def module_names(cls, config) -> list[str]:
        names = ["embed_tokens", "rotary_emb"]
        if decoder_spec(config).local_rope:
            names.append("rotary_emb_local")
        names += [f"layers.{i}" for i in range(config.num_hidden_layers)]
        names.append("norm")
        return names

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_parallel_context(self, pc: ParallelContext):
        self.pc = pc
        for layer in self.layers:
            if not is_released(layer):
                layer.self_attn.pc = pc
                if layer.self_attn.spec.qk_norm and pc is not None and pc.tp_size > 1:
                    # q_norm / k_norm weights are shared by all heads but see only this rank's heads
                    layer.self_attn.q_norm.grad_sum_group = pc.tp_group
                    layer.self_attn.k_norm.grad_sum_group = pc.tp_group

    def _mark_partial_grad_norms(self, group) -> None:
        """Under token-sharded tensor parallelism a norm weight sees 1/tp of the tokens on each rank: its gradient is a
        partial sum.  The optimizer adds the parts over ``group`` once per step (``FusedAdamW._reduce_partial_grads``)."""
        if getattr(self, "_partial_marked", None) is group:
            return
        norms = [self.norm] if self.holds("norm") else []
        for layer in self.layers:
            if not is_released(layer):
                norms += [layer.input_layernorm, layer.post_attention_layernorm]
        for n in norms:
            n.weight.tp_partial_grad_group = group
        self._partial_marked = group

    def embed(self, input_ids, feats=None, src=None):
        h = self.embed_tokens(input_ids, feats, src)
        if self.spec.embed_scale:
            h = h * (self.config.hidden_size ** 0.5)
        return h

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, position_ids=None, hidden_states=None,
                **kwargs):
        first = self.holds("embed_tokens")
        if hidden_states is None:
            if inputs_embeds is None:
                assert first, "this stage has no embedding: pass hidden_states"
                inputs_embeds = self.embed(input_ids)
            hidden_states = inputs_embeds
        B, S, _ = hidden_states.shape
        # Token-sharded tensor parallelism: between the parallel blocks every rank holds the rows [r T/tp, (r+1) T/tp) of
        # the flattened [B*S, H] activations.  The first stage takes its rows of the (replicated) embeddings; a later
        # stage receives its rows from the same tensor-parallel rank of the stage before it.
        tp_shard = None
        if self.pc is not None and self.pc.tp_seq_shard:
            from ..ops import _native as nat

            Bf, Sf = kwargs.get("full_shape") or (B, S)
            incoming_shard = B * S != Bf * Sf
            grp = None if nat.LIBRARY_MODE else self.pc.seq_shard_group(Bf * Sf, hidden_states)
            if grp is not None and not all(l.supports_seq_shard() for l in self.layers if not is_released(l)):
                grp = None
            assert grp is not None or not incoming_shard, "received token-sharded activations but this stage cannot shard"
            if grp is not None:
                if not incoming_shard:
                    hidden_states = comm.split_forward_gather_backward(hidden_states.reshape(1, B * S, -1), 1, grp)
                tp_shard = (Bf, Sf, grp)
                B, S = Bf, Sf
                self._mark_partial_grad_norms(grp)
        mask = as_attn_mask(attention_mask, B, S, hidden_states.device)
        pos = position_ids
        cp_state = None
        if self.pc is not None and self.pc.sp_mode == "ring_attn" and self.pc.sp_size > 1:
            hidden_states, pos, mask, cp_state, S_full = self._context_parallel_split(hidden_states, mask, kwargs)
            B, S, _ = hidden_states.shape
            kwargs = dict(kwargs, rope_len=max(int(kwargs.get("rope_len", 0) or 0), S_full))
        elif self.pc is not None and self.pc.sp_mode == "all_to_all" and self.pc.sp_size > 1 and first:
            # Ulysses: every rank keeps a contiguous 1/sp slice of the sequence between attention layers
            hidden_states = comm.split_forward_gather_backward(hidden_states, 1, self.pc.sp_group, 1.0 / self.pc.sp_size)
        # positions beyond max_position_embeddings (context-parallel shards of a long sequence) need `rope_len`
        max_pos = max(S, int(kwargs.get("rope_len", 0) or 0))
        rope = self.rotary_emb(hidden_states.device, max_pos)
        delta, residual = hidden_states, None
        aux_losses = []
        recompute = self.gradient_checkpointing and self.training and torch.is_grad_enabled()
        n_recompute = sum(not is_released(l) for l in self.layers) - int(getattr(self, "recompute_keep_layers", 0))
        seen = 0
        for layer in self.layers:
            if is_released(layer):
                continue
            seen += 1
            lrope = rope
            if self.spec.local_rope and getattr(self.config, "layer_types", None):
                if self.config.layer_types[layer.self_attn.layer_idx] == "sliding_attention":
                    lrope = self.rotary_emb_local(hidden_states.device, max_pos)
            grad_sync_layer_input(layer, delta)
            if recompute and seen <= n_recompute:
                delta, residual, aux = checkpoint_layer(layer, delta, residual, lrope, pos, mask, tp_shard)
            else:
                delta, residual, aux = layer(delta, residual, lrope, pos, mask, tp_shard)
            if aux is not None:
                aux_losses.append(aux)
        if self.holds("norm"):
            if residual is None:
                out = self.norm(delta)
            else:
                out, _ = self.norm(delta, residual)
            if self.pc is not None and self.pc.sp_mode == "all_to_all" and self.pc.sp_size > 1:
                # Ulysses: back to the full sequence for the LM head (the loss is computed identically on every sp rank)
                out = comm.gather_forward_split_backward(out, 1, self.pc.sp_group, float(self.pc.sp_size))
            if tp_shard is not None:
                # the LM head (vocab-parallel, or replicated) works on all tokens again
                out = comm.gather_forward_split_backward(out, 1, tp_shard[2]).view(B, S, -1)
        else:
            out = delta if residual is None else delta + residual
        return ModelOutput(last_hidden_state=out, router_logits=tuple(aux_losses) if aux_losses else None, cp_state=cp_state)

    def _context_parallel_split(self, hidden_states, mask, kwargs):
        """Pick this rank's tokens (first stage) and express the mask through global positions."""
        from ..parallel.cp import ContextParallelBatchSplitUtils as U, ContextParallelState

        B, S, _ = hidden_states.shape
        S_full = mask.q_bits.shape[1] if mask.q_bits is not None else int(kwargs.get("full_seq_len", 0) or S)
        offsets = U.create_context_parallel_split(mask if mask.q_bits is not None else None, self.pc.sp_group,
                                                  self.pc.cp_dist_mode, seq_len=S_full, batch=B, device=hidden_states.device)
        if offsets is None:
            return hidden_states, None, mask, None, S_full
        state = ContextParallelState(self.pc.sp_group, offsets, mask, hidden_states.device)
        if S == S_full:
            hidden_states = hidden_states.index_select(1, state.mine)
        pos = state.mine.int()[None].expand(B, -1).contiguous()
        return hidden_states, pos, state.local_mask, state, S_full


def _full_seq_len(kwargs, input_ids, labels) -> int:
    """Length of the whole sequence as a later pipeline stage can know it under context parallelism: its hidden states
    hold this rank's tokens only, but the micro-batch still carries the full ``input_ids`` / ``labels``."""
    n = kwargs.get("full_seq_len")
    if n:
        return int(n)
    for t in (input_ids, labels):
        if t is not None:
            return int(t.shape[1])
    return 0


def _full_shape(kwargs, input_ids, labels):
    """``(batch, sequence length)`` of the whole micro-batch as a later pipeline stage can know it when its hidden states
    hold only this rank's token rows (token-sharded tensor parallelism): given explicitly, or from ``input_ids`` / ``labels``."""
    fs = kwargs.get("full_shape")
    if fs:
        return tuple(int(v) for v in fs)
    for t in (input_ids, labels):
        if t is not None and t.dim() == 2:
            return int(t.shape[0]), int(t.shape[1])
    return None


def as_attn_mask(attention_mask, B: int, S: int, device) -> A.AttnMask:
    """Accept ``None`` (causal), an :class:`AttnMask`, an int64 bitfield ``[B,S]`` or a 0/1 padding mask ``[B,S]``."""
    if attention_mask is None:
        return A.AttnMask.causal()
    if isinstance(attention_mask, A.AttnMask):
        return attention_mask
    m = attention_mask
    if m.dtype == torch.int64 and m.dim() == 2 and bool((m > 1).any()):
        return A.AttnMask.bitfield(m)
    # padding mask: valid tokens become text tokens of a bitfield mask (causal + padding)
    bits = torch.where(m.bool(), torch.full_like(m, (1 << 62) | 1, dtype=torch.int64), torch.zeros_like(m, dtype=torch.int64))
    return A.AttnMask.bitfield(bits)


class DecoderForCausalLM(PreTrainedModel):
    """``LlamaForCausalLM``-shaped model: ``model.*`` + ``lm_head`` with the fused LM-head cross-entropy."""

    config_class = DecoderConfig
    base_model_prefix = "model"

    def __init__(self, config):
        super().__init__(config)
        self.model = DecoderModel(config)
        self.lm_head = cnn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if getattr(config, "tie_word_embeddings", False):
            self.lm_head.weight = self.model.embed_tokens.weight
        self.vocab_start = 0  # first vocabulary id of the local LM-head shard under tensor parallelism
        self.pc: ParallelContext | None = None

    @classmethod
    def module_names(cls, config) -> list[str]:
        return [f"model.{n}" for n in DecoderModel.module_names(config)] + ["lm_head"]

    def hold_only(self, names):
        super().hold_only(names)
        self.model._held = {n[len("model."):] for n in names if n.startswith("model.")}

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def set_parallel_context(self, pc: ParallelContext):
        self.pc = pc
        self.model.set_parallel_context(pc)

    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs=None):
        super().gradient_checkpointing_enable(gradient_checkpointing_kwargs)
        self.model.gradient_checkpointing = True
        self.model.recompute_keep_layers = self.recompute_keep_layers

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, position_ids=None, labels=None,
                hidden_states=None, return_logits: bool | None = None, shift_labels: bool = True, **kwargs):
        out = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, attention_mask=attention_mask,
                         position_ids=position_ids, hidden_states=hidden_states, rope_len=kwargs.get("rope_len", 0),
                         full_seq_len=_full_seq_len(kwargs, input_ids, labels), full_shape=_full_shape(kwargs, input_ids, labels))
        h = out.last_hidden_state
        if not self.holds("lm_head"):
            return ModelOutput(hidden_states=h, router_logits=out.router_logits)
        result = ModelOutput(router_logits=out.router_logits)
        tp_group = self.pc.tp_group if self.pc is not None else None
        softcap = self.model.spec.final_softcap
        cp_state = out.get("cp_state")
        if labels is not None and not softcap:
            tgt = labels
            if shift_labels:
                tgt = torch.full_like(labels, -100)
                tgt[:, :-1] = labels[:, 1:]
            if cp_state is not None and cp_state.mine is not None and tgt.shape[1] != h.shape[1]:
                tgt = tgt.index_select(1, cp_state.mine)
            w = self.lm_head.weight
            valid = getattr(self, "valid_vocab", None)
            if valid is not None and valid < w.shape[0]:
                w = w[:valid]  # rows beyond the real vocabulary are padding of the vocab-parallel shard
            h_in = comm.reduce_backward(h, tp_group) if tp_group is not None else h  # each vocab shard yields a partial dh
            loss_sum, n_valid = linear_cross_entropy(h_in, w, tgt, tp_group=tp_group,
                                                     vocab_start=self.vocab_start, reduction="sum_and_count")
            if cp_state is not None:
                # every context-parallel rank sees a token subset: normalise by the global token count and
                # pre-multiply by sp so that the dp x sp gradient average yields d(sum / count)
                total = n_valid.clone().float()
                torch.distributed.all_reduce(total, group=cp_state.group)
                sp = torch.distributed.get_world_size(cp_state.group)
                result["loss_sum"], result["num_valid"] = loss_sum, total
                result["loss"] = loss_sum * sp / total.clamp(min=1).to(loss_sum.dtype)
            else:
                result["loss_sum"], result["num_valid"] = loss_sum, n_valid
                result["loss"] = loss_sum / n_valid.clamp(min=1).to(loss_sum.dtype)
        if return_logits or (labels is None) or softcap:
            logits = linear(comm.reduce_backward(h, tp_group) if tp_group is not None else h, self.lm_head.weight)
            tp_sharded = tp_group is not None and comm._world(tp_group) > 1
            # the soft-capped loss below is a plain cross-entropy over the whole vocabulary: gather the shards for it
            keep_sharded = tp_sharded and bool(self.pc and self.pc.parallel_output and labels is not None) and not softcap
            if tp_sharded and not keep_sharded:
                logits = comm.gather_forward_split_backward(logits, logits.dim() - 1, tp_group)
                full_v = getattr(self.lm_head, "full_vocab_size", None)
                if full_v is not None and full_v < logits.shape[-1]:
                    logits = logits[..., :full_v]  # drop the padding rows of the vocab-parallel shards
            if softcap:
                logits = torch.tanh(logits / softcap) * softcap
                if labels is not None:
                    tgt = labels
                    if shift_labels:
                        tgt = torch.full_like(labels, -100)
                        tgt[:, :-1] = labels[:, 1:]
                    if cp_state is not None and cp_state.mine is not None and tgt.shape[1] != h.shape[1]:
                        tgt = tgt.index_select(1, cp_state.mine)
                    lf = logits.float().view(-1, logits.shape[-1])
                    loss_sum = torch.nn.functional.cross_entropy(lf, tgt.reshape(-1), ignore_index=-100, reduction="sum")
                    n_valid = (tgt != -100).sum()
                    if cp_state is not None:
                        total = n_valid.clone().float()
                        torch.distributed.all_reduce(total, group=cp_state.group)
                        sp = torch.distributed.get_world_size(cp_state.group)
                        result["loss_sum"], result["num_valid"] = loss_sum, total
                        result["loss"] = loss_sum * sp / total.clamp(min=1).to(loss_sum.dtype)
                    else:
                        result["loss_sum"], result["num_valid"] = loss_sum, n_valid
                        result["loss"] = loss_sum / n_valid.clamp(min=1)
            result["logits"] = logits
        return result


LlamaModel = DecoderModel
LlamaForCausalLM = DecoderForCausalLM

for _mt, _cfg in (("llama", LlamaConfig), ("mistral", MistralConfig), ("qwen2", Qwen2Config), ("qwen3", Qwen3Config),
                  ("gemma", GemmaConfig), ("gemma2", Gemma2Config), ("gemma3_text", Gemma3TextConfig), ("phi3", Phi3Config)):
    register_model(_mt, _cfg, DecoderForCausalLM)
