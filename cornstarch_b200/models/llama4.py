"""Llama-4 text decoder (dense + MoE layers) with HF parameter names.

What differs from the Llama family handled by :mod:`.llama` (reference: cornstarch/shardformer/modeling/llama4.py:458-582,
policy cornstarch/shardformer/policies/llama4.py:40-51,188-218):

* rotary embedding on interleaved pairs (complex multiplication), skipped on the "NoPE" layers (``no_rope_layers``);
* weight-less L2 norm of q and k after the rotation on the RoPE layers (``use_qk_norm``);
* temperature tuning of the queries on NoPE layers: ``q *= log1p(floor((pos + 1) / floor_scale)) * attn_scale + 1``;
* MoE layers (``moe_layers``): sigmoid router scores of the top-k experts scale the expert INPUT, the experts' weights
  are stacked (``experts.gate_up_proj [E, H, 2I]``, ``experts.down_proj [E, I, H]``, stored input-major, which the GEMM
  reads as is), and a shared expert runs on every token; the other layers use a dense MLP of ``intermediate_size_mlp``.

Chunked attention (``attention_chunk_size``) equals causal attention for sequences up to the chunk size, which is what
this module supports; longer sequences are rejected.  Pipeline units: ``model.embed_tokens, model.rotary_emb,
model.layers.i, model.norm, lm_head``.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import nn as cnn
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.cross_entropy import linear_cross_entropy
from ..ops.gemm import gemm
from ..ops.linear import linear, multi_linear
from ..parallel import comm
from ..utils.recompute import checkpoint_layer
from .base import ModelOutput, PreTrainedModel, is_released, register_model
from .llama import DecoderConfig


class Llama4TextConfig(DecoderConfig):
    model_type = "llama4_text"

    def __init__(self, intermediate_size_mlp=16384, num_local_experts=16, num_experts_per_tok=1, interleave_moe_layer_step=1,
                 moe_layers=None, no_rope_layers=None, use_qk_norm=True, attn_temperature_tuning=True, floor_scale=8192,
                 attn_scale=0.1, attention_chunk_size=8192, router_aux_loss_coef=0.001, **kw):
        kw.setdefault("rms_norm_eps", 1e-5)
        kw.setdefault("rope_theta", 500000.0)
        rp = kw.pop("rope_parameters", None)
        if rp and "rope_theta" in rp:
            kw["rope_theta"] = rp["rope_theta"]
        kw.pop("layer_types", None)
        super().__init__(**kw)
        L = self.num_hidden_layers
        self.intermediate_size_mlp = intermediate_size_mlp
        self.num_local_experts, self.num_experts_per_tok = num_local_experts, num_experts_per_tok
        self.interleave_moe_layer_step = interleave_moe_layer_step
        self.moe_layers = list(moe_layers) if moe_layers is not None else list(
            range(interleave_moe_layer_step - 1, L, interleave_moe_layer_step))
        self.no_rope_layers = list(no_rope_layers) if no_rope_layers else [int((i + 1) % 4 != 0) for i in range(L)]
        self.use_qk_norm, self.attn_temperature_tuning = use_qk_norm, attn_temperature_tuning
        self.floor_scale, self.attn_scale, self.attention_chunk_size = floor_scale, attn_scale, attention_chunk_size
        self.router_aux_loss_coef = router_aux_loss_coef


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs ``(x[2i], x[2i+1])`` by the angle of frequency ``i`` (``cos``/``sin``: ``[S, D/2]``)."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    out = torch.stack([xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c], dim=-1)
    return out.flatten(-2).to(x.dtype)


class _InputMajorLinearFn(torch.autograd.Function):
    """``y = x W`` with ``W`` stored ``[in, out]``; forward, dX and dW all read the operands as stored."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        return gemm(x2, w, False, True)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = dy.contiguous()
        return gemm(dy, w, False, False), gemm(x2, dy, True, True, out_dtype=w.dtype)


class Llama4TextExperts(nn.Module):
    def __init__(self, config):
        super().__init__()
        E_, H, I = config.num_local_experts, config.hidden_size, config.intermediate_size
        self.gate_up_proj = nn.Parameter(torch.empty(E_, H, 2 * I).normal_(std=0.02))
        self.down_proj = nn.Parameter(torch.empty(E_, I, H).normal_(std=0.02))
        self.act = config.hidden_act

    def run(self, e: int, x2: torch.Tensor) -> torch.Tensor:
        gu = _InputMajorLinearFn.apply(x2, self.gate_up_proj[e])
        return _InputMajorLinearFn.apply(E.glu(gu, self.act), self.down_proj[e])


class _Router(nn.Module):
    def __init__(self, H, n):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n, H).normal_(std=0.02))


class _DenseMLP(nn.Module):
    def __init__(self, H, I, act):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = cnn.Linear(H, I, bias=False), cnn.Linear(H, I, bias=False), cnn.Linear(I, H, bias=False)
        self.act = act

    def forward(self, x):
        gu = multi_linear(self.gate_proj.input_hook(x), [self.gate_proj.weight, self.up_proj.weight], tp=self.gate_proj.tp_spec(x))
        return self.down_proj(E.glu(gu, self.act))


class Llama4TextMoe(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.top_k, self.num_experts = config.num_experts_per_tok, config.num_local_experts
        self.experts = Llama4TextExperts(config)
        self.router = _Router(config.hidden_size, self.num_experts)
        self.shared_expert = _DenseMLP(config.hidden_size, config.intermediate_size, config.hidden_act)

    def forward(self, x):
        B, S, H = x.shape
        x2 = x.reshape(-1, H)
        logits = linear(x2, self.router.weight)
        top_v, top_i = torch.topk(logits.float(), self.top_k, dim=-1)
        scores = torch.sigmoid(top_v).to(x2.dtype)  # [T, k]; experts outside the top-k get score 0, i.e. a zero input
        flat_e = top_i.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        token_of = torch.div(order, self.top_k, rounding_mode="floor")
        counts = torch.bincount(flat_e, minlength=self.num_experts).tolist()
        xin = x2[token_of] * scores.reshape(-1)[order].unsqueeze(-1)
        outs, start = [], 0
        for e, n in enumerate(counts):
            if n:
                outs.append(self.experts.run(e, xin[start : start + n]))
            start += n
        routed = torch.zeros_like(x2)
        if outs:
            routed.index_add_(0, token_of, torch.cat(outs, dim=0))
        return (self.shared_expert(x2) + routed).view(B, S, H), logits


class Llama4TextAttention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        H, D = config.hidden_size, config.head_dim
        self.head_dim, self.num_heads, self.num_kv_heads = D, config.num_attention_heads, config.num_key_value_heads
        self.use_rope = bool(config.no_rope_layers[layer_idx])
        self.qk_norm = bool(config.use_qk_norm) and self.use_rope
        self.temperature = bool(config.attn_temperature_tuning) and not self.use_rope
        self.floor_scale, self.attn_scale, self.eps = config.floor_scale, config.attn_scale, config.rms_norm_eps
        self.chunk = int(config.attention_chunk_size)  # RoPE layers attend causally inside chunks of this many tokens
        bias = bool(config.attention_bias)
        self.q_proj = cnn.Linear(H, self.num_heads * D, bias=bias)
        self.k_proj = cnn.Linear(H, self.num_kv_heads * D, bias=bias)
        self.v_proj = cnn.Linear(H, self.num_kv_heads * D, bias=bias)
        self.o_proj = cnn.Linear(self.num_heads * D, H, bias=bias)
        self.attn_impl = None

    def forward(self, x, rope, pos, mask):
        B, S, _ = x.shape
        D, Hq, Hk = self.head_dim, self.num_heads, self.num_kv_heads
        qkv = multi_linear(self.q_proj.input_hook(x), [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight],
                           [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias] if self.q_proj.bias is not None else None,
                           tp=self.q_proj.tp_spec(x))
        q, k, v = qkv[..., : Hq * D], qkv[..., Hq * D : (Hq + Hk) * D], qkv[..., (Hq + Hk) * D :]
        pc = getattr(self, "pc", None)
        ulysses = pc is not None and pc.sp_mode == "all_to_all" and pc.sp_size > 1
        if ulysses:
            # [B, S/sp, heads * D] -> [B, S, heads/sp * D]: from here to the output projection every rank sees the whole
            # sequence for its share of the heads, so rotary positions, temperature and chunking need no bookkeeping
            q, k, v = (comm.all_to_all_comm(t.contiguous(), pc.sp_group, 2, 1) for t in (q, k, v))
            Hq, Hk, S = Hq // pc.sp_size, Hk // pc.sp_size, q.shape[1]
        q, k, v = q.reshape(B, S, Hq, D), k.reshape(B, S, Hk, D), v.reshape(B, S, Hk, D)
        ring = getattr(mask, "_cp_state", None) is not None  # this rank holds the tokens at global positions `pos`
        if self.use_rope:
            cos, sin = (rope[0][:S], rope[1][:S]) if pos is None else (rope[0].index_select(0, pos), rope[1].index_select(0, pos))
            q, k = rope_interleaved(q, cos, sin), rope_interleaved(k, cos, sin)
        if self.qk_norm:
            q = (q.float() * torch.rsqrt(q.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
            k = (k.float() * torch.rsqrt(k.float().pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        if self.temperature:
            p = torch.arange(S, device=x.device, dtype=torch.float32) if pos is None else pos.float()
            scales = torch.log1p(torch.floor((p + 1.0) / self.floor_scale)) * self.attn_scale + 1.0
            q = (q * scales.view(1, S, 1, 1)).to(x.dtype)
        fn = self.attn_impl or A.attention
        if self.use_rope and S > self.chunk and not ring:
            # chunked attention: chunks are independent causal sequences, i.e. further batch entries (the tail is padded
            # with keys that no real query can see, because they come after every real token of their chunk)
            assert mask is None or mask.mode == A.MASK_CAUSAL, "chunked attention supports the plain causal mask"
            C = self.chunk
            pad = (-S) % C
            if pad:
                q, k, v = (F.pad(t, (0, 0, 0, 0, 0, pad)) for t in (q, k, v))
            n = (S + pad) // C
            q, k, v = (t.reshape(B * n, C, t.shape[2], D).contiguous() for t in (q, k, v))
            o = fn(q, k, v, A.AttnMask.causal(), None).reshape(B, n * C, Hq, D)[:, :S]
        else:
            o = fn(q.contiguous(), k.contiguous(), v.contiguous(), mask, None)
        o = o.reshape(B, S, Hq * D)
        if ulysses:
            o = comm.all_to_all_comm(o, pc.sp_group, 1, 2)  # back to [B, S/sp, all heads * D]
        return self.o_proj(o)


class Llama4TextDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.self_attn = Llama4TextAttention(config, layer_idx)
        self.is_moe = layer_idx in config.moe_layers
        self.feed_forward = Llama4TextMoe(config) if self.is_moe else _DenseMLP(config.hidden_size, config.intermediate_size_mlp, config.hidden_act)
        self.input_layernorm = cnn.RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.post_attention_layernorm = cnn.RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, x, rope, pos, mask):
        a = self.self_attn(self.input_layernorm(x), rope, pos, mask)
        h, x = self.post_attention_layernorm(a, x)  # x <- x + a; h = norm(x)
        out = self.feed_forward(h)
        m, logits = out if isinstance(out, tuple) else (out, None)
        return x + m, logits


class _Rotary(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dim, self.theta = config.head_dim, config.rope_theta
        self._t = None

    def tables(self, n, device):
        if self._t is None or self._t[0].shape[0] < n or self._t[0].device != torch.device(device):
            self._t = E.rope_tables(n, self.dim, self.theta, device)
        return self._t


class Llama4TextModel(PreTrainedModel):
    config_class = Llama4TextConfig

    def __init__(self, config):
        super().__init__(config)
        self.embed_tokens = cnn.Embedding(config.vocab_size, config.hidden_size)
        self.rotary_emb = _Rotary(config)
        self.layers = nn.ModuleList([Llama4TextDecoderLayer(config, i) for i in range(config.num_hidden_layers)])
        self.norm = cnn.RMSNorm(config.hidden_size, config.rms_norm_eps)

    @classmethod
    def module_names(cls, config):
        return ["embed_tokens", "rotary_emb"] + [f"layers.{i}" for i in range(config.num_hidden_layers)] + ["norm"]

    def get_input_embeddings(self):
        return self.embed_tokens

    def set_parallel_context(self, pc):
        self.pc = pc
        for layer in self.layers:
            if not is_released(layer):
                layer.self_attn.pc = pc

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, hidden_states=None, **kw):
        from .llama import as_attn_mask

        if hidden_states is None:
            hidden_states = inputs_embeds if inputs_embeds is not None else self.embed_tokens(input_ids)
        pc = getattr(self, "pc", None)
        ulysses = pc is not None and pc.sp_mode == "all_to_all" and pc.sp_size > 1
        if ulysses:
            assert attention_mask is None, "Ulysses for Llama-4 supports the plain causal mask"
            if self.holds("embed_tokens"):
                # every rank keeps a contiguous 1/sp slice of the sequence between attention layers
                hidden_states = comm.split_forward_gather_backward(hidden_states, 1, pc.sp_group, 1.0 / pc.sp_size)
        B, S, _ = hidden_states.shape
        mask = as_attn_mask(attention_mask, B, S, hidden_states.device)
        pos, chunk_mask, cp_state, S_full = None, None, None, S
        if pc is not None and pc.sp_mode == "ring_attn" and pc.sp_size > 1:
            assert attention_mask is None, "ring attention for Llama-4 supports the plain causal mask"
            hidden_states, pos, mask, chunk_mask, cp_state, S_full = self._context_parallel_split(hidden_states, kw)
            S = hidden_states.shape[1]
        rope = self.rotary_emb.tables(S_full * (pc.sp_size if ulysses else 1), hidden_states.device)
        x, router = hidden_states, []
        for layer in self.layers:
            if is_released(layer):
                continue
            m = chunk_mask if (chunk_mask is not None and layer.self_attn.use_rope) else mask
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x, lg = checkpoint_layer(layer, x, rope, pos, m)
            else:
                x, lg = layer(x, rope, pos, m)
            if lg is not None:
                router.append(lg)
        if is_released(self.norm):
            return ModelOutput(hidden_states=x, router_logits=tuple(router) or None, cp_state=cp_state)
        out = self.norm(x)
        if ulysses:
            # back to the full sequence for the LM head (the loss is then the same on every sequence-parallel rank)
            out = comm.gather_forward_split_backward(out, 1, pc.sp_group, float(pc.sp_size))
        return ModelOutput(last_hidden_state=out, router_logits=tuple(router) or None, cp_state=cp_state)

    def _context_parallel_split(self, hidden_states, kw):
        """Ring attention: pick this rank's tokens (on the first stage) and state both masks through global positions.

        The global (NoPE) layers use the causal mask.  The chunked layers use a bitfield mask: a query carries the text
        bit and the bit of its chunk, a key only the bit of its chunk, so a query sees the earlier keys of its own chunk.
        One bit per chunk limits a sequence to 60 chunks.  The reference runs this model under ring attention too
        (cornstarch/shardformer/modeling/llama4.py:148-200)."""
        from ..parallel.cp import ContextParallelBatchSplitUtils as U, ContextParallelState

        pc, dev = self.pc, hidden_states.device
        B, S, _ = hidden_states.shape
        first = self.holds("embed_tokens")
        S_full = int(kw.get("full_seq_len") or (S if first else S * pc.sp_size))
        offsets = U.create_context_parallel_split(None, pc.sp_group, pc.cp_dist_mode, seq_len=S_full, batch=B, device=dev)
        if offsets is None:  # too short to split: every rank computes the whole sequence
            return hidden_states, None, A.AttnMask.causal(), None, None, S_full
        state = ContextParallelState(pc.sp_group, offsets, A.AttnMask.causal(), dev)
        chunk_mask, C = None, int(self.config.attention_chunk_size)
        if S_full > C:
            n_chunks = (S_full + C - 1) // C
            assert n_chunks <= 60, f"{n_chunks} attention chunks: ring attention for Llama-4 encodes at most 60 in its mask"
            chunk_bit = torch.ones(B, S_full, dtype=torch.int64, device=dev) << (1 + torch.arange(S_full, device=dev) // C)
            chunk_state = ContextParallelState(pc.sp_group, offsets, A.AttnMask.bitfield(chunk_bit | 1, k_bits=chunk_bit), dev)
            chunk_mask = chunk_state.local_mask
        if S == S_full and first:
            hidden_states = hidden_states.index_select(1, state.mine)
        return hidden_states, state.mine.int(), state.local_mask, chunk_mask, state, S_full


class Llama4ForCausalLM(PreTrainedModel):
    config_class = Llama4TextConfig

    def __init__(self, config):
        super().__init__(config)
        self.model = Llama4TextModel(config)
        self.lm_head = cnn.Linear(config.hidden_size, config.vocab_size, bias=False)
        self.vocab_start = 0    # first vocabulary id of the local LM-head shard under tensor parallelism
        self.valid_vocab = None  # rows of the local shard that are real vocabulary (the rest is padding)
        self.tp_group = None

    def set_parallel_context(self, pc):
        self.tp_group = pc.tp_group if pc is not None else None
        if hasattr(self.model, "set_parallel_context"):
            self.model.set_parallel_context(pc)

    @classmethod
    def module_names(cls, config):
        return [f"model.{n}" for n in Llama4TextModel.module_names(config)] + ["lm_head"]

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        self.model.gradient_checkpointing = self.gradient_checkpointing
        from .llama import _full_seq_len

        out = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, attention_mask=attention_mask, hidden_states=hidden_states,
                         full_seq_len=_full_seq_len(kw, input_ids, labels))
        if "last_hidden_state" not in out or not self.holds("lm_head"):
            return ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")), router_logits=out.router_logits)
        h = out.last_hidden_state
        res = ModelOutput(last_hidden_state=h, router_logits=out.router_logits)
        if labels is not None:
            tgt = torch.full_like(labels, -100)
            tgt[:, :-1] = labels[:, 1:]
            w = self.lm_head.weight
            if self.valid_vocab is not None and self.valid_vocab < w.shape[0]:
                w = w[: self.valid_vocab]
            tp = self.tp_group if (self.tp_group is not None and comm._world(self.tp_group) > 1) else None
            h_in = comm.reduce_backward(h, tp) if tp is not None else h  # each vocabulary shard yields a partial dh
            cp_state = out.get("cp_state")
            if cp_state is not None:
                # this rank holds a token subset: normalise by the global token count, pre-multiplied by sp so that
                # the gradient average over the dp x sp group yields d(sum / count)
                tgt = tgt.index_select(1, cp_state.mine)
                loss_sum, n_valid = linear_cross_entropy(h_in, w, tgt, tp_group=tp, vocab_start=self.vocab_start,
                                                         reduction="sum_and_count")
                total = n_valid.clone().float()
                torch.distributed.all_reduce(total, group=cp_state.group)
                sp = torch.distributed.get_world_size(cp_state.group)
                res["loss_sum"], res["num_valid"] = loss_sum, total
                res["loss"] = loss_sum * sp / total.clamp(min=1).to(loss_sum.dtype)
            else:
                res["loss"] = linear_cross_entropy(h_in, w, tgt, tp_group=tp, vocab_start=self.vocab_start)
        else:
            tp = self.tp_group if (self.tp_group is not None and comm._world(self.tp_group) > 1) else None
            logits = linear(comm.reduce_backward(h, tp) if tp is not None else h, self.lm_head.weight)
            res["logits"] = comm.gather_forward_split_backward(logits, logits.dim() - 1, tp) if tp is not None else logits
        return res


register_model("llama4_text", Llama4TextConfig, Llama4ForCausalLM)
