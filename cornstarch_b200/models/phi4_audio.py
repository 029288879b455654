"""Phi-4-multimodal audio encoder (conformer blocks) with HF parameter names.

Pipeline units as in the reference's policy (cornstarch/shardformer/policies/phi4_multimodal.py:37-47):
``encoder_embedding, embed, relative_attention_bias_layer, encoders.i``.  Block structure (patched forward
cornstarch/shardformer/modeling/phi4_multimodal.py): half-step GLU feed-forward, self-attention with a learned
relative-position bias per head, a convolution module (point-wise GLU conv, depth-wise separable conv, point-wise
conv), second half-step feed-forward, final LayerNorm.

Linear layers, LayerNorms and the GLU run on this package's kernels.  The attention adds a dense ``[heads, T, T]``
bias to the scores, which the flash-attention kernels of this package do not take, so it goes through PyTorch's
scaled-dot-product attention; the audio sequences are short (T = frames / time_reduction), and the 1-D / 2-D
convolutions use cuDNN through PyTorch like the other front-ends.

Parallel forms: tensor parallelism splits the heads and both feed-forwards (every rank reads its heads' columns of the
replicated bias table); Ulysses ("all_to_all") splits the tokens between the attention layers and the heads inside
them; under context parallelism ("ring_attn") the tokens are split in contiguous chunks after the
sub-sampling front-end, keys / values are gathered, each rank keeps the bias rows of its own queries and the causal
depth-wise convolutions fetch their ``kernel_size - 1`` left neighbours from the previous rank; a later pipeline stage
receives the bias together with the hidden states.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import nn as cnn
from ..ops import elementwise as E
from ..parallel import comm
from ..ops.linear import multi_linear
from ..utils.recompute import checkpoint_layer
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, is_released, register_model


class Phi4MultimodalAudioConfig(PretrainedConfig):
    model_type = "phi4_multimodal_audio"
    composite_key = "audio_config"

    def __init__(self, hidden_size=1024, intermediate_size=1536, num_blocks=24, num_attention_heads=16, activation="swish",
                 chunk_size=-1, left_chunk=18, conv_activation="swish", conv_glu_type="swish", depthwise_multiplier=1,
                 depthwise_separable_out_channel=1024, ext_pw_out_channel=1024, input_size=80, kernel_size=3,
                 nemo_conv_channels=1024, nemo_final_size=None, time_reduction=8, bias_max_distance=1000, bias_symmetric=False,
                 nemo_activation="relu", **kw):
        self.hidden_size, self.intermediate_size, self.num_blocks = hidden_size, intermediate_size, num_blocks
        self.num_attention_heads, self.activation = num_attention_heads, activation
        self.conv_activation, self.conv_glu_type, self.depthwise_multiplier = conv_activation, conv_glu_type, depthwise_multiplier
        self.depthwise_separable_out_channel, self.ext_pw_out_channel = depthwise_separable_out_channel, ext_pw_out_channel
        self.input_size, self.kernel_size, self.nemo_conv_channels, self.time_reduction = input_size, kernel_size, nemo_conv_channels, time_reduction
        self.bias_max_distance, self.bias_symmetric, self.nemo_activation = bias_max_distance, bias_symmetric, nemo_activation
        self.chunk_size, self.left_chunk = chunk_size, left_chunk
        if nemo_final_size is None:
            length = input_size
            for _ in range(int(math.log2(time_reduction))):
                length = math.floor((length - 1) / 2 + 1)
            nemo_final_size = length
        self.nemo_final_size = nemo_final_size
        kw.pop("depthwise_seperable_out_channel", None)
        super().__init__(**kw)

    num_hidden_layers = property(lambda self: self.num_blocks)


_ACT = {"swish": "silu", "silu": "silu", "relu": "relu", "gelu": "gelu"}


class _MeanVarNorm(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.register_buffer("global_mean", torch.zeros(config.input_size))
        self.register_buffer("global_invstd", torch.ones(config.input_size))

    def forward(self, x):
        return (x - self.global_mean.to(x.dtype)) * self.global_invstd.to(x.dtype)


class _NemoConvSubsampling(nn.Module):
    def __init__(self, config):
        super().__init__()
        c = config.nemo_conv_channels
        act = nn.ReLU() if config.nemo_activation == "relu" else nn.SiLU()
        layers = [nn.Conv2d(1, c, 3, 2, 1), act]
        for _ in range(int(math.log2(config.time_reduction)) - 1):
            layers += [nn.Conv2d(c, c, 3, 2, 1, groups=c), nn.Conv2d(c, c, 1, 1, 0), act]
        self.conv = nn.Sequential(*layers)
        self.out = cnn.Linear(c * config.nemo_final_size, config.hidden_size)

    def forward(self, x):
        h = self.conv(x.unsqueeze(1).to(self.conv[0].weight.dtype))
        b, _, t, _ = h.shape
        return self.out(h.transpose(1, 2).reshape(b, t, -1))


class _RelativeAttentionBias(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.max_distance, self.symmetric = config.bias_max_distance, config.bias_symmetric
        self.num_buckets = self.max_distance * (1 if self.symmetric else 2)
        self.bias_values = nn.Embedding(self.num_buckets, config.num_attention_heads)
        # groups that split the heads, outermost first, as (group, sum_gradient): tensor parallelism (the table is
        # replicated and its gradient summed over the ranks) and then Ulysses sequence parallelism (no sum: the
        # gradients of sequence-parallel ranks are partial sums like those of every other parameter)
        self.head_splits: list = []

    def forward(self, T: int, device, rows: tuple[int, int] | None = None):
        """``rows = (start, end)``: only the bias of those query positions (a context-parallel rank's tokens)."""
        pos = torch.arange(T, device=device)
        q_pos = pos if rows is None else pos[rows[0] : rows[1]]
        rel = (pos[None, :] - q_pos[:, None]).clamp(-self.max_distance, self.max_distance - 1)
        idx = rel.abs() if self.symmetric else rel + self.num_buckets // 2
        w = self.bias_values.weight
        for group, sum_gradient in self.head_splits:
            n, r = comm._world(group), torch.distributed.get_rank(group)
            per = w.shape[1] // n
            w = (comm.reduce_backward(w, group) if sum_gradient else w)[:, r * per : (r + 1) * per]
        return F.embedding(idx, w).permute(2, 0, 1).unsqueeze(0)  # [1, local heads, T or rows, T]


class _AudioMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer_norm = cnn.LayerNorm(config.hidden_size, 1e-5)
        self.gate_up_proj = cnn.Linear(config.hidden_size, 2 * config.intermediate_size)
        self.down_proj = cnn.Linear(config.intermediate_size, config.hidden_size)
        self.act = _ACT[config.activation]

    def forward(self, x):
        up, gate = self.gate_up_proj(self.layer_norm(x)).chunk(2, dim=-1)  # HF order: value first, gate second
        return self.down_proj(E.glu(torch.cat([gate, up], dim=-1), self.act))


def _cp_sizes(T: int, world: int) -> list[int]:
    """Tokens per rank of ``torch.tensor_split(T tokens, world)``."""
    return [T // world + (1 if r < T % world else 0) for r in range(world)]


class _AudioAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads, self.head_dim = config.num_attention_heads, H // config.num_attention_heads
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = cnn.Linear(H, H), cnn.Linear(H, H), cnn.Linear(H, H), cnn.Linear(H, H)
        self.cp_group = None  # context parallelism: x holds this rank's tokens, the bias its rows against all keys
        self.ulysses_group = None  # Ulysses: x holds this rank's tokens; attention sees all tokens for a share of the heads

    def forward(self, x, bias):
        B, T, _ = x.shape
        W, heads = self.num_heads * self.head_dim, self.num_heads
        qkv = multi_linear(self.q_proj.input_hook(x), [self.q_proj.weight, self.k_proj.weight, self.v_proj.weight],
                           [self.q_proj.bias, self.k_proj.bias, self.v_proj.bias])
        q, k, v = (qkv[..., i * W : (i + 1) * W] for i in range(3))
        ulysses = self.ulysses_group is not None and comm._world(self.ulysses_group) > 1
        if ulysses:
            q, k, v = (comm.all_to_all_comm(t.contiguous(), self.ulysses_group, 2, 1) for t in (q, k, v))  # [B, T_all, W / sp]
            heads, T = heads // comm._world(self.ulysses_group), q.shape[1]
        q, k, v = (t.reshape(B, T, heads, self.head_dim).transpose(1, 2) for t in (q, k, v))
        if self.cp_group is not None and comm._world(self.cp_group) > 1:
            kv = comm.gather_forward_reduce_scatter_backward(torch.stack([k, v]), 3, self.cp_group,
                                                             _cp_sizes(bias.shape[-1], comm._world(self.cp_group)))
            k, v = kv[0], kv[1]
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype))
        o = o.transpose(1, 2).reshape(B, T, heads * self.head_dim)
        if ulysses:
            o = comm.all_to_all_comm(o, self.ulysses_group, 1, 2)  # back to [B, T_local, W]
        return self.o_proj(o)


class _GluPointWiseConv(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.out_dim = config.ext_pw_out_channel
        self.ext_pw_conv_1d = nn.Conv1d(config.hidden_size, 2 * self.out_dim, 1)
        self.b1 = nn.Parameter(torch.zeros(1, self.out_dim, 1))
        self.b2 = nn.Parameter(torch.zeros(1, self.out_dim, 1))
        self.act = _ACT[config.conv_glu_type]

    def forward(self, x):  # [B, T, H] -> [B, T, out]: a 1x1 convolution is a linear layer over channels
        w = self.ext_pw_conv_1d.weight.squeeze(-1)
        h = cnn.linear(x, w, self.ext_pw_conv_1d.bias)
        a = h[..., : self.out_dim] + self.b1.view(1, 1, -1).to(h.dtype)
        g = h[..., self.out_dim :] + self.b2.view(1, 1, -1).to(h.dtype)
        return E.glu(torch.cat([g, a], dim=-1), self.act)


class _DepthWiseSeparableConv1d(nn.Module):
    def __init__(self, config, padding):
        super().__init__()
        H = config.hidden_size
        self.dw_conv = nn.Conv1d(H, H * config.depthwise_multiplier, config.kernel_size, 1, padding=padding, groups=H)
        self.pw_conv = nn.Conv1d(H * config.depthwise_multiplier, config.depthwise_separable_out_channel, 1)

    def forward(self, x):
        return self.pw_conv(self.dw_conv(x))


class _ConvModule(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.kernel_size = config.kernel_size
        self.layer_norm = cnn.LayerNorm(config.hidden_size, 1e-5)
        self.glu = _GluPointWiseConv(config)
        self.dw_sep_conv_1d = _DepthWiseSeparableConv1d(config, padding=config.kernel_size - 1)
        self.ext_pw_conv_1d = nn.Conv1d(config.hidden_size, config.ext_pw_out_channel, 1)
        self.act = _ACT[config.conv_activation]
        self.cp_group = None

    def forward(self, x):
        h = self.glu(self.layer_norm(x)).permute(0, 2, 1)
        conv = self.dw_sep_conv_1d
        h = h.to(conv.dw_conv.weight.dtype)
        if self.cp_group is not None and comm._world(self.cp_group) > 1 and self.kernel_size > 1:
            # the causal convolution looks kernel_size - 1 tokens back: they come from the previous rank, and the
            # depth-wise convolution then runs without padding
            h = comm.halo_from_previous(h, 2, self.kernel_size - 1, self.cp_group)
            dw = conv.dw_conv
            h = conv.pw_conv(F.conv1d(h, dw.weight, dw.bias, 1, 0, 1, dw.groups))
        else:
            h = conv(h)
            if self.kernel_size > 1:
                h = h[:, :, : -(self.kernel_size - 1)]  # causal: drop the look-ahead the symmetric padding added
        h = E.activation(h.permute(0, 2, 1).contiguous(), self.act)
        return cnn.linear(h, self.ext_pw_conv_1d.weight.squeeze(-1), self.ext_pw_conv_1d.bias)


class Phi4MultimodalAudioConformerEncoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.feed_forward_in = _AudioMLP(config)
        self.self_attn = _AudioAttention(config)
        self.conv = _ConvModule(config)
        self.feed_forward_out = _AudioMLP(config)
        self.layer_norm_att = cnn.LayerNorm(config.hidden_size, 1e-5)
        self.layer_norm = cnn.LayerNorm(config.hidden_size, 1e-5)

    def forward(self, x, bias):
        r = x + 0.5 * self.feed_forward_in(x)
        x = r + self.self_attn(self.layer_norm_att(r), bias)
        x = x + self.conv(x)
        x = x + 0.5 * self.feed_forward_out(x)
        return self.layer_norm(x)


class Phi4MultimodalAudioModel(PreTrainedModel):
    config_class = Phi4MultimodalAudioConfig
    main_input_name = "audio_input_features"

    def __init__(self, config):
        super().__init__(config)
        self.encoder_embedding = _MeanVarNorm(config)
        self.embed = _NemoConvSubsampling(config)
        self.relative_attention_bias_layer = _RelativeAttentionBias(config)
        self.encoders = nn.ModuleList([Phi4MultimodalAudioConformerEncoderLayer(config) for _ in range(config.num_blocks)])

    @classmethod
    def module_names(cls, config):
        return ["encoder_embedding", "embed", "relative_attention_bias_layer"] + [f"encoders.{i}" for i in range(config.num_blocks)]

    def set_parallel_context(self, pc):
        self.pc = pc
        sp = pc.sp_group if pc is not None and pc.sp_mode in ("ring_attn", "all_to_all") and pc.sp_size > 1 else None
        ring = sp if pc is not None and pc.sp_mode == "ring_attn" else None
        ulysses = sp if pc is not None and pc.sp_mode == "all_to_all" else None
        self._cp_group, self._ulysses_group = ring, ulysses
        for layer in self.encoders:
            if not is_released(layer):
                layer.self_attn.cp_group, layer.self_attn.ulysses_group = ring, ulysses
                layer.conv.cp_group = sp  # the tokens are split in contiguous chunks in both modes
        if not is_released(self.relative_attention_bias_layer):
            splits = [(pc.tp_group, True)] if pc is not None and pc.tp_size > 1 else []
            self.relative_attention_bias_layer.head_splits = splits + ([(ulysses, False)] if ulysses is not None else [])

    def forward(self, audio_input_features=None, hidden_states=None, attention_bias=None, **kw):
        """A later pipeline stage gets ``hidden_states`` and the ``attention_bias`` the first stage computed (the
        reference hands its ``attention_mask`` on the same way, cornstarch/shardformer/modeling/phi4_multimodal.py:148-189)."""
        if hidden_states is None:
            x = self.embed(self.encoder_embedding(audio_input_features))
        else:
            x = hidden_states
        bias = attention_bias
        if bias is None:
            cp, ul, T = getattr(self, "_cp_group", None), getattr(self, "_ulysses_group", None), x.shape[1]
            if ul is not None:
                # Ulysses: equal contiguous chunks between the attention layers; attention sees every token, so the bias
                # keeps all rows (of this rank's heads)
                assert T % comm._world(ul) == 0, f"{T} audio tokens do not divide over {comm._world(ul)} sequence-parallel ranks"
                x = comm.split_forward_gather_backward(x, 1, ul)
                bias = self.relative_attention_bias_layer(T, x.device)
            elif cp is None:
                bias = self.relative_attention_bias_layer(T, x.device)
            else:
                # context parallelism: contiguous token chunks in rank order (the causal convolutions need their left
                # neighbours), every rank keeps the bias rows of its own tokens
                sizes, r = _cp_sizes(T, comm._world(cp)), torch.distributed.get_rank(cp)
                x = comm.split_forward_gather_backward(x, 1, cp)
                bias = self.relative_attention_bias_layer(T, x.device, rows=(sum(sizes[:r]), sum(sizes[: r + 1])))
        for layer in self.encoders:
            if is_released(layer):
                continue
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint_layer(layer, x, bias)
            else:
                x = layer(x, bias)
        if is_released(self.encoders[-1]):
            return ModelOutput(hidden_states=x, attention_bias=bias)
        return ModelOutput(last_hidden_state=x)


register_model("phi4_multimodal_audio", Phi4MultimodalAudioConfig, Phi4MultimodalAudioModel)
