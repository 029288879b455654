"""GPT-2, BERT and OPT with HF parameter names on the fused kernels.

These are the language models of the heterogeneous-pipeline examples of the reference
(examples/pipeline_template/run_{gpt2,bert}.py) and of its thin policies
(cornstarch/shardformer/policies/{gpt2,bert,opt}.py: ``get_all_modules`` :44-55, :57-71, :35-48).
Every model follows the pipeline protocol of this package: ``module_names(config)`` lists the
pipeline-assignable units in order, ``hold_only`` releases the rest, a non-first stage is called with
``hidden_states=`` and a non-last stage returns ``ModelOutput(hidden_states=...)``.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from ..utils.recompute import checkpoint_layer

from .. import nn as cnn
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.cross_entropy import linear_cross_entropy
from ..ops.gemm import gemm
from ..ops.linear import linear, multi_linear
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, is_released, register_model


def _padding_mask(attention_mask, causal: bool) -> A.AttnMask:
    """0/1 padding mask -> kernel mask (valid tokens = text bit; causal order or full visibility among valid tokens)."""
    if attention_mask is None:
        return A.AttnMask.causal() if causal else A.AttnMask.full()
    m = attention_mask
    if causal:
        bits = torch.where(m.bool(), torch.full_like(m, (1 << 62) | 1, dtype=torch.int64), torch.zeros_like(m, dtype=torch.int64))
    else:
        # one shared modality bit: every valid token sees every valid token
        bits = torch.where(m.bool(), torch.full_like(m, 2, dtype=torch.int64), torch.zeros_like(m, dtype=torch.int64))
    return A.AttnMask.bitfield(bits)


def _run_layers(layers, x, mask, ckpt: bool):
    for layer in layers:
        if is_released(layer):
            continue
        x = checkpoint_layer(layer, x, mask) if (ckpt and torch.is_grad_enabled()) else layer(x, mask)
    return x


def _lm_loss(h, weight, labels, shift: bool):
    tgt = labels
    if shift:
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
    return linear_cross_entropy(h, weight, tgt)


# ------------------------------------------------------------------------------------------------ GPT-2
class GPT2Config(PretrainedConfig):
    model_type = "gpt2"

    def __init__(self, vocab_size=50257, n_positions=1024, n_embd=768, n_layer=12, n_head=12, n_inner=None,
                 activation_function="gelu_new", layer_norm_epsilon=1e-5, tie_word_embeddings=True, **kw):
        self.vocab_size, self.n_positions, self.n_embd, self.n_layer, self.n_head = vocab_size, n_positions, n_embd, n_layer, n_head
        self.n_inner = n_inner
        self.activation_function = activation_function
        self.layer_norm_epsilon = layer_norm_epsilon
        self.tie_word_embeddings = tie_word_embeddings
        super().__init__(**kw)

    hidden_size = property(lambda self: self.n_embd)
    num_hidden_layers = property(lambda self: self.n_layer)
    num_attention_heads = property(lambda self: self.n_head)


class _Conv1DFn(torch.autograd.Function):
    """``y = x W + b`` with ``W`` stored ``[in, out]`` (GPT-2 checkpoints); all three GEMMs read W as stored."""

    @staticmethod
    def forward(ctx, x2, w, b):
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        return gemm(x2, w, False, True, bias=b)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, False, False)                # [T,out] x [in,out]^T
        dw = gemm(x2, dy, True, True, out_dtype=w.dtype)  # x^T dy -> [in,out]
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return dx, dw, db


class Conv1D(nn.Module):
    """GPT-2's linear layer with the weight stored ``[in, out]``.  ``shard`` makes the tensor-parallel variants: ``"col"``
    keeps a slice of the output features (per fused part when ``split_sizes`` is given), ``"row"`` a slice of the input
    features with the partial results summed over the group."""

    def __init__(self, nf: int, nx: int):
        super().__init__()
        self.nf, self.nx = nf, nx
        self.weight = nn.Parameter(torch.empty(nx, nf).normal_(std=0.02))
        self.bias = nn.Parameter(torch.zeros(nf))
        self.process_group, self.parallel, self.split_sizes = None, None, None

    @classmethod
    def shard(cls, module: "Conv1D", process_group, kind: str, split_sizes: list[int] | None = None) -> "Conv1D":
        import torch.distributed as dist

        tp, r = dist.get_world_size(process_group), dist.get_rank(process_group)
        w, b = module.weight.data, module.bias.data
        if kind == "col":
            lw = cnn.shard_rows(w.t(), tp, r, split_sizes).t().contiguous()
            lb = cnn.shard_rows(b, tp, r, split_sizes).clone()
        else:
            lw, lb = cnn.shard_rows(w, tp, r).clone(), b.clone()
        new = cls.__new__(cls)
        nn.Module.__init__(new)
        new.nx, new.nf = lw.shape
        new.weight = nn.Parameter(lw, requires_grad=module.weight.requires_grad)
        new.bias = nn.Parameter(lb, requires_grad=module.bias.requires_grad)
        new.process_group, new.parallel, new.split_sizes = process_group, kind, split_sizes
        return new

    def forward(self, x):
        from ..parallel import comm

        if self.parallel == "col":
            x = comm.reduce_backward(x, self.process_group)
        row = self.parallel == "row"
        y = _Conv1DFn.apply(x.reshape(-1, self.nx), self.weight, None if row else self.bias)
        y = y.view(*x.shape[:-1], self.nf)
        if row:
            y = comm.reduce_forward(y, self.process_group) + self.bias.to(y.dtype)
        return y


class _GPT2Attention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_attn = Conv1D(3 * config.n_embd, config.n_embd)
        self.c_proj = Conv1D(config.n_embd, config.n_embd)


class _GPT2MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        inner = config.n_inner or 4 * config.n_embd
        self.c_fc = Conv1D(inner, config.n_embd)
        self.c_proj = Conv1D(config.n_embd, inner)


class GPT2Block(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.num_heads, self.head_dim = config.n_head, config.n_embd // config.n_head
        self.act = config.activation_function
        self.ln_1 = cnn.LayerNorm(config.n_embd, config.layer_norm_epsilon)
        self.attn = _GPT2Attention(config)
        self.ln_2 = cnn.LayerNorm(config.n_embd, config.layer_norm_epsilon)
        self.mlp = _GPT2MLP(config)

    def forward(self, x, mask):
        B, S, H = x.shape
        qkv = self.attn.c_attn(self.ln_1(x)).view(B, S, 3, self.num_heads, self.head_dim)
        a = A.attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], mask)
        a = self.attn.c_proj(a.reshape(B, S, self.num_heads * self.head_dim))
        h2, x = self.ln_2(a, x)
        return x + self.mlp.c_proj(E.activation(self.mlp.c_fc(h2), self.act))


class GPT2Model(PreTrainedModel):
    config_class = GPT2Config

    def __init__(self, config):
        super().__init__(config)
        self.wte = cnn.Embedding(config.vocab_size, config.n_embd)
        self.wpe = cnn.Embedding(config.n_positions, config.n_embd)
        self.drop = nn.Identity()
        self.h = nn.ModuleList([GPT2Block(config) for _ in range(config.n_layer)])
        self.ln_f = cnn.LayerNorm(config.n_embd, config.layer_norm_epsilon)

    @classmethod
    def module_names(cls, config):
        return ["wte", "wpe", "drop"] + [f"h.{i}" for i in range(config.n_layer)] + ["ln_f"]

    def forward(self, input_ids=None, attention_mask=None, hidden_states=None, position_ids=None, **kw):
        if hidden_states is None:
            S = input_ids.shape[1]
            pos = position_ids if position_ids is not None else torch.arange(S, device=input_ids.device)[None]
            hidden_states = self.wte(input_ids) + self.wpe(pos)
        x = _run_layers(self.h, hidden_states, _padding_mask(attention_mask, True), self.gradient_checkpointing and self.training)
        if is_released(self.ln_f):
            return ModelOutput(hidden_states=x)
        return ModelOutput(last_hidden_state=self.ln_f(x))


class GPT2LMHeadModel(PreTrainedModel):
    config_class = GPT2Config

    def __init__(self, config):
        super().__init__(config)
        self.transformer = GPT2Model(config)
        self.lm_head = cnn.Linear(config.n_embd, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.transformer.wte.weight

    @classmethod
    def module_names(cls, config):
        return [f"transformer.{n}" for n in GPT2Model.module_names(config)] + ["lm_head"]

    def get_input_embeddings(self):
        return self.transformer.wte

    def forward(self, input_ids=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        self.transformer.gradient_checkpointing = self.gradient_checkpointing
        out = self.transformer(input_ids=input_ids, attention_mask=attention_mask, hidden_states=hidden_states, **kw)
        if "last_hidden_state" not in out or not self.holds("lm_head"):
            return ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        h = out.last_hidden_state
        res = ModelOutput(last_hidden_state=h)
        if labels is not None:
            res["loss"] = _lm_loss(h, self.lm_head.weight, labels, True)
        else:
            res["logits"] = linear(h, self.lm_head.weight)
        return res


# ------------------------------------------------------------------------------------------------ BERT
class BertConfig(PretrainedConfig):
    model_type = "bert"

    def __init__(self, vocab_size=30522, hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072,
                 hidden_act="gelu", max_position_embeddings=512, type_vocab_size=2, layer_norm_eps=1e-12,
                 tie_word_embeddings=True, **kw):
        self.vocab_size, self.hidden_size, self.num_hidden_layers = vocab_size, hidden_size, num_hidden_layers
        self.num_attention_heads, self.intermediate_size, self.hidden_act = num_attention_heads, intermediate_size, hidden_act
        self.max_position_embeddings, self.type_vocab_size, self.layer_norm_eps = max_position_embeddings, type_vocab_size, layer_norm_eps
        self.tie_word_embeddings = tie_word_embeddings
        super().__init__(**kw)


class BertEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.word_embeddings = cnn.Embedding(config.vocab_size, H)
        self.position_embeddings = cnn.Embedding(config.max_position_embeddings, H)
        self.token_type_embeddings = cnn.Embedding(config.type_vocab_size, H)
        self.LayerNorm = cnn.LayerNorm(H, config.layer_norm_eps)

    def forward(self, input_ids, token_type_ids=None):
        S = input_ids.shape[1]
        pos = torch.arange(S, device=input_ids.device)[None]
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        return self.LayerNorm(self.word_embeddings(input_ids) + self.position_embeddings(pos) + self.token_type_embeddings(tt))


class _BertSelf(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.query, self.key, self.value = cnn.Linear(H, H), cnn.Linear(H, H), cnn.Linear(H, H)


class _BertOut(nn.Module):
    def __init__(self, i, o, eps):
        super().__init__()
        self.dense = cnn.Linear(i, o)
        self.LayerNorm = cnn.LayerNorm(o, eps)


class _BertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self = _BertSelf(config.hidden_size)
        self.output = _BertOut(config.hidden_size, config.hidden_size, config.layer_norm_eps)


class _BertIntermediate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = cnn.Linear(config.hidden_size, config.intermediate_size)


class BertLayer(nn.Module):
    """Post-LN block: ``x = LN(x + attn(x)); x = LN(x + mlp(x))``."""

    def __init__(self, config):
        super().__init__()
        self.num_heads, self.head_dim, self.act = config.num_attention_heads, config.hidden_size // config.num_attention_heads, config.hidden_act
        self.attention = _BertAttention(config)
        self.intermediate = _BertIntermediate(config)
        self.output = _BertOut(config.intermediate_size, config.hidden_size, config.layer_norm_eps)

    def forward(self, x, mask):
        B, S, _ = x.shape
        s = self.attention.self
        W = self.num_heads * self.head_dim
        qkv = multi_linear(s.query.input_hook(x), [s.query.weight, s.key.weight, s.value.weight], [s.query.bias, s.key.bias, s.value.bias])
        q, k, v = (qkv[..., i * W : (i + 1) * W].view(B, S, self.num_heads, self.head_dim) for i in range(3))
        a = self.attention.output.dense(A.attention(q, k, v, mask).reshape(B, S, W))
        x, _ = self.attention.output.LayerNorm(a, x)  # LN(x + a)
        m = self.output.dense(E.activation(self.intermediate.dense(x), self.act))
        x, _ = self.output.LayerNorm(m, x)
        return x


class _BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])


class _BertPooler(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = cnn.Linear(config.hidden_size, config.hidden_size)

    def forward(self, x):
        return torch.tanh(self.dense(x[:, 0]))


class BertModel(PreTrainedModel):
    config_class = BertConfig

    def __init__(self, config, add_pooling_layer=True):
        super().__init__(config)
        self.embeddings = BertEmbeddings(config)
        self.encoder = _BertEncoder(config)
        self.pooler = _BertPooler(config) if add_pooling_layer else None
        self._has_pooler = add_pooling_layer
        self.causal = bool(getattr(config, "is_decoder", False))  # BertLMHeadModel as a decoder attends causally

    @classmethod
    def module_names(cls, config, add_pooling_layer=True):
        return ["embeddings"] + [f"encoder.layer.{i}" for i in range(config.num_hidden_layers)] + (["pooler"] if add_pooling_layer else [])

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, hidden_states=None, **kw):
        if hidden_states is None:
            hidden_states = self.embeddings(input_ids, token_type_ids)
        x = _run_layers(self.encoder.layer, hidden_states, _padding_mask(attention_mask, self.causal),
                        self.gradient_checkpointing and self.training)
        last_held = not is_released(self.encoder.layer[-1])
        if not last_held:
            return ModelOutput(hidden_states=x)
        pooled = self.pooler(x) if (self.pooler is not None and not is_released(self.pooler)) else None
        return ModelOutput(last_hidden_state=x, pooler_output=pooled)


class _BertTransform(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = cnn.Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.act = config.hidden_act

    def forward(self, x):
        return self.LayerNorm(E.activation(self.dense(x), self.act))


class _BertPredictions(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.transform = _BertTransform(config)
        self.decoder = cnn.Linear(config.hidden_size, config.vocab_size, bias=True)
        self.bias = self.decoder.bias


class _BertMLMHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.predictions = _BertPredictions(config)


class BertForMaskedLM(PreTrainedModel):
    config_class = BertConfig

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=False)
        self.cls = _BertMLMHead(config)
        if config.tie_word_embeddings:
            self.cls.predictions.decoder.weight = self.bert.embeddings.word_embeddings.weight

    @classmethod
    def module_names(cls, config):
        return [f"bert.{n}" for n in BertModel.module_names(config, False)] + ["cls"]

    def get_input_embeddings(self):
        return self.bert.embeddings.word_embeddings

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, **kw):
        self.bert.gradient_checkpointing = self.gradient_checkpointing
        out = self.bert(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids, hidden_states=hidden_states)
        if "last_hidden_state" not in out or not self.holds("cls"):
            return ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        p = self.cls.predictions
        logits = linear(p.transform(out.last_hidden_state), p.decoder.weight, p.decoder.bias)
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), labels.reshape(-1), ignore_index=-100)
        return res


# ------------------------------------------------------------------------------------------------ OPT
class OPTConfig(PretrainedConfig):
    model_type = "opt"

    def __init__(self, vocab_size=50272, hidden_size=768, num_hidden_layers=12, ffn_dim=3072, num_attention_heads=12,
                 max_position_embeddings=2048, activation_function="relu", do_layer_norm_before=True, word_embed_proj_dim=None,
                 enable_bias=True, layer_norm_elementwise_affine=True, tie_word_embeddings=True, **kw):
        self.vocab_size, self.hidden_size, self.num_hidden_layers, self.ffn_dim = vocab_size, hidden_size, num_hidden_layers, ffn_dim
        self.num_attention_heads, self.max_position_embeddings = num_attention_heads, max_position_embeddings
        self.activation_function, self.do_layer_norm_before = activation_function, do_layer_norm_before
        self.word_embed_proj_dim = word_embed_proj_dim or hidden_size
        self.enable_bias, self.layer_norm_elementwise_affine = enable_bias, layer_norm_elementwise_affine
        self.tie_word_embeddings = tie_word_embeddings
        super().__init__(**kw)


class _OPTAttention(nn.Module):
    def __init__(self, H, bias):
        super().__init__()
        self.k_proj, self.v_proj = cnn.Linear(H, H, bias=bias), cnn.Linear(H, H, bias=bias)
        self.q_proj, self.out_proj = cnn.Linear(H, H, bias=bias), cnn.Linear(H, H, bias=bias)


class OPTDecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads, self.head_dim = config.num_attention_heads, H // config.num_attention_heads
        self.act, self.pre_ln = config.activation_function, config.do_layer_norm_before
        self.self_attn = _OPTAttention(H, config.enable_bias)
        self.self_attn_layer_norm = cnn.LayerNorm(H, 1e-5)
        self.fc1 = cnn.Linear(H, config.ffn_dim, bias=config.enable_bias)
        self.fc2 = cnn.Linear(config.ffn_dim, H, bias=config.enable_bias)
        self.final_layer_norm = cnn.LayerNorm(H, 1e-5)

    def forward(self, x, mask):
        B, S, _ = x.shape
        a = self.self_attn
        W = self.num_heads * self.head_dim
        h = self.self_attn_layer_norm(x) if self.pre_ln else x
        biases = [a.q_proj.bias, a.k_proj.bias, a.v_proj.bias] if a.q_proj.bias is not None else None
        qkv = multi_linear(a.q_proj.input_hook(h), [a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], biases)
        q, k, v = (qkv[..., i * W : (i + 1) * W].view(B, S, self.num_heads, self.head_dim) for i in range(3))
        o = a.out_proj(A.attention(q, k, v, mask).reshape(B, S, W))
        if self.pre_ln:
            h2, x = self.final_layer_norm(o, x)
            return x + self.fc2(E.activation(self.fc1(h2), self.act))
        x, _ = self.self_attn_layer_norm(o, x)
        m = self.fc2(E.activation(self.fc1(x), self.act))
        x, _ = self.final_layer_norm(m, x)
        return x


class OPTDecoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        H, P = config.hidden_size, config.word_embed_proj_dim
        self.embed_tokens = cnn.Embedding(config.vocab_size, P)
        self.embed_positions = cnn.Embedding(config.max_position_embeddings + 2, H)  # learned positions with offset 2
        self.project_in = cnn.Linear(P, H, bias=False) if P != H else None
        self.project_out = cnn.Linear(H, P, bias=False) if P != H else None
        self.final_layer_norm = cnn.LayerNorm(H, 1e-5) if config.do_layer_norm_before else None
        self.layers = nn.ModuleList([OPTDecoderLayer(config) for _ in range(config.num_hidden_layers)])


class OPTModel(PreTrainedModel):
    config_class = OPTConfig

    def __init__(self, config):
        super().__init__(config)
        self.decoder = OPTDecoder(config)

    @classmethod
    def module_names(cls, config):
        proj = (config.word_embed_proj_dim or config.hidden_size) != config.hidden_size
        names = ["decoder.embed_tokens", "decoder.embed_positions"] + (["decoder.project_in"] if proj else [])
        names += [f"decoder.layers.{i}" for i in range(config.num_hidden_layers)]
        names += (["decoder.final_layer_norm"] if config.do_layer_norm_before else []) + (["decoder.project_out"] if proj else [])
        return names

    def forward(self, input_ids=None, attention_mask=None, hidden_states=None, **kw):
        d = self.decoder
        if hidden_states is None:
            S = input_ids.shape[1]
            if attention_mask is not None:
                pos = (torch.cumsum(attention_mask, dim=1) * attention_mask).long() - 1 + 2
            else:
                pos = torch.arange(S, device=input_ids.device)[None] + 2
            x = d.embed_tokens(input_ids)
            if d.project_in is not None:
                x = d.project_in(x)
            hidden_states = x + d.embed_positions(pos.clamp(min=0))
        x = _run_layers(d.layers, hidden_states, _padding_mask(attention_mask, True), self.gradient_checkpointing and self.training)
        if is_released(d.layers[-1]):
            return ModelOutput(hidden_states=x)
        if d.final_layer_norm is not None and not is_released(d.final_layer_norm):
            x = d.final_layer_norm(x)
        if d.project_out is not None and not is_released(d.project_out):
            x = d.project_out(x)
        return ModelOutput(last_hidden_state=x)


class OPTForCausalLM(PreTrainedModel):
    config_class = OPTConfig

    def __init__(self, config):
        super().__init__(config)
        self.model = OPTModel(config)
        self.lm_head = cnn.Linear(config.word_embed_proj_dim, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.decoder.embed_tokens.weight

    @classmethod
    def module_names(cls, config):
        return [f"model.{n}" for n in OPTModel.module_names(config)] + ["lm_head"]

    def get_input_embeddings(self):
        return self.model.decoder.embed_tokens

    def forward(self, input_ids=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        self.model.gradient_checkpointing = self.gradient_checkpointing
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, hidden_states=hidden_states)
        if "last_hidden_state" not in out or not self.holds("lm_head"):
            return ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        h = out.last_hidden_state
        res = ModelOutput(last_hidden_state=h)
        if labels is not None:
            res["loss"] = _lm_loss(h, self.lm_head.weight, labels, True)
        else:
            res["logits"] = linear(h, self.lm_head.weight)
        return res


register_model("gpt2", GPT2Config, GPT2LMHeadModel)
register_model("bert", BertConfig, BertForMaskedLM)
register_model("opt", OPTConfig, OPTForCausalLM)
