"""Whisper-style audio encoders (Whisper, Qwen2-Audio) with HF parameter names on the fused kernels.

Front-end: two 1-D convolutions over the log-mel spectrogram (the second with stride 2) + fixed
sinusoidal positions; then pre-LN transformer blocks (``k_proj`` has no bias) and a final LayerNorm.
Module names per pipeline unit follow cornstarch/shardformer/policies/whisper.py:36-47 and
policies/qwen2_audio.py:39-50; the patched forwards they replace are
cornstarch/shardformer/modeling/{whisper,qwen2_audio}.py.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from ..utils.recompute import checkpoint_layer

from .. import nn as cnn
from ..ops import attention as A
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, is_released, register_model
from .vision import _SelfAttn, encoder_block


class WhisperConfig(PretrainedConfig):
    model_type = "whisper"

    def __init__(self, num_mel_bins=80, d_model=384, encoder_layers=4, encoder_attention_heads=6, encoder_ffn_dim=1536,
                 max_source_positions=1500, activation_function="gelu", encoder_layerdrop=0.0, layer_norm_eps=1e-5, **kw):
        self.num_mel_bins = num_mel_bins
        self.d_model = d_model
        self.encoder_layers = encoder_layers
        self.encoder_attention_heads = encoder_attention_heads
        self.encoder_ffn_dim = encoder_ffn_dim
        self.max_source_positions = max_source_positions
        self.activation_function = activation_function
        self.encoder_layerdrop = encoder_layerdrop
        self.layer_norm_eps = layer_norm_eps
        super().__init__(**kw)

    @property
    def hidden_size(self):
        return self.d_model

    @property
    def num_hidden_layers(self):
        return self.encoder_layers

    def to_dict(self):
        d = super().to_dict()
        return d


class Qwen2AudioEncoderConfig(WhisperConfig):
    composite_key = "audio_config"  # nested under this name in a Qwen2-Audio checkpoint's config.json
    model_type = "qwen2_audio_encoder"


class WhisperEncoderLayer(nn.Module):
    """HF names: ``self_attn.{q,k,v,out}_proj``, ``self_attn_layer_norm``, ``fc1``, ``fc2``, ``final_layer_norm``."""

    def __init__(self, config):
        super().__init__()
        H = config.d_model
        self.act = config.activation_function
        self.self_attn = _SelfAttn(H, config.encoder_attention_heads, bias=True, k_bias=False)
        self.self_attn_layer_norm = cnn.LayerNorm(H, config.layer_norm_eps)
        self.fc1 = cnn.Linear(H, config.encoder_ffn_dim)
        self.fc2 = cnn.Linear(config.encoder_ffn_dim, H)
        self.final_layer_norm = cnn.LayerNorm(H, config.layer_norm_eps)

    def forward(self, x, mask):
        a = self.self_attn
        return encoder_block(x, self.self_attn_layer_norm, a.q_proj, a.k_proj, a.v_proj, a.out_proj,
                             self.final_layer_norm, self.fc1, self.fc2, self.act, a.num_heads, mask, a.attn_impl)


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


class WhisperEncoder(PreTrainedModel):
    config_class = WhisperConfig
    main_input_name = "input_features"
    has_avg_pooler = False

    def __init__(self, config):
        super().__init__(config)
        H = config.d_model
        self.conv1 = nn.Conv1d(config.num_mel_bins, H, kernel_size=3, padding=1)
        self.conv2 = nn.Conv1d(H, H, kernel_size=3, stride=2, padding=1)
        self.embed_positions = nn.Embedding(config.max_source_positions, H)
        with torch.no_grad():
            if self.embed_positions.weight.device.type != "meta":
                self.embed_positions.weight.copy_(sinusoids(config.max_source_positions, H))
        self.embed_positions.weight.requires_grad_(False)
        self.layers = nn.ModuleList([WhisperEncoderLayer(config) for _ in range(config.encoder_layers)])
        self.layer_norm = cnn.LayerNorm(H, config.layer_norm_eps)
        if self.has_avg_pooler:
            self.avg_pooler = nn.AvgPool1d(2, stride=2)
        self.layerdrop = config.encoder_layerdrop

    @classmethod
    def module_names(cls, config):
        names = ["conv1", "conv2", "embed_positions"] + [f"layers.{i}" for i in range(config.encoder_layers)] + ["layer_norm"]
        if cls.has_avg_pooler:
            names.append("avg_pooler")
        return names

    def embed(self, input_features):
        w = self.conv1.weight
        x = F.gelu(self.conv1(input_features.to(w.dtype)))
        x = F.gelu(self.conv2(x)).permute(0, 2, 1)
        return x + self.embed_positions.weight[: x.shape[1]].to(x.dtype)

    def forward(self, input_features=None, hidden_states=None, **kw):
        if hidden_states is None:
            assert self.holds("conv1"), "this stage has no front-end: pass hidden_states"
            hidden_states = self.embed(input_features)
            if getattr(self, "_cp_group", None) is not None:
                from ..parallel import comm

                hidden_states = comm.split_forward_gather_backward(hidden_states, 1, self._cp_group)
        x = hidden_states
        mask = A.AttnMask.full()
        if getattr(self, "_cp_group", None) is not None:
            from ..parallel.cp import ContextParallelState

            mask = ContextParallelState(self._cp_group, None, None, x.device).local_mask
        for layer in self.layers:
            if is_released(layer):
                continue
            if self.training and self.layerdrop > 0 and torch.rand(()) < self.layerdrop:
                continue  # LayerDrop, kept from the reference (cornstarch/shardformer/modeling/whisper.py:108-116)
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint_layer(layer, x, mask)
            else:
                x = layer(x, mask)
        if not self.holds("layer_norm"):
            return ModelOutput(hidden_states=x)
        if self.has_avg_pooler:
            x = self.avg_pooler(x.permute(0, 2, 1)).permute(0, 2, 1)
        return ModelOutput(last_hidden_state=self.layer_norm(x))


class Qwen2AudioEncoder(WhisperEncoder):
    config_class = Qwen2AudioEncoderConfig
    has_avg_pooler = True


register_model("whisper", WhisperConfig, WhisperEncoder)
register_model("qwen2_audio_encoder", Qwen2AudioEncoderConfig, Qwen2AudioEncoder)
