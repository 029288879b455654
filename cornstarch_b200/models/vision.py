"""Vision encoders (SigLIP, CLIP, ViT) with HF parameter names on the fused kernels.

Each family differs only in its embedding front-end, module names and activation; the transformer
block is shared (:class:`EncoderLayerCore`): LayerNorm -> fused q|k|v GEMM (+bias) -> full (bidirectional)
flash attention -> out-proj -> residual+LayerNorm fused -> fc1 -> GELU -> fc2.  Head dims that are not
multiples of 16 (SigLIP-so400m: 72) are handled inside the attention kernel by zero-padded TMA boxes.

Replaces the patched HF forwards of cornstarch/shardformer/modeling/{siglip,clip,vit}.py and the module
lists of cornstarch/shardformer/policies/{siglip,clip,vit}.py (names returned by ``module_names``).
"""

from __future__ import annotations


import torch
import torch.nn as nn
from ..utils.recompute import checkpoint_layer

from .. import nn as cnn
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.linear import multi_linear
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, is_released, register_model


class VisionConfig(PretrainedConfig):
    composite_key = "vision_config"

    model_type = "siglip_vision_model"

    def __init__(self, hidden_size=768, intermediate_size=3072, num_hidden_layers=12, num_attention_heads=12,
                 num_channels=3, image_size=224, patch_size=16, hidden_act="gelu_pytorch_tanh", layer_norm_eps=1e-6,
                 attention_dropout=0.0, **kw):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_hidden_layers = num_hidden_layers
        self.num_attention_heads = num_attention_heads
        self.num_channels = num_channels
        self.image_size = image_size
        self.patch_size = patch_size
        self.hidden_act = hidden_act
        self.layer_norm_eps = layer_norm_eps
        self.attention_dropout = attention_dropout
        super().__init__(**kw)


class SiglipVisionConfig(VisionConfig):
    model_type = "siglip_vision_model"


class CLIPVisionConfig(VisionConfig):
    model_type = "clip_vision_model"

    def __init__(self, **kw):
        kw.setdefault("hidden_act", "quick_gelu")
        kw.setdefault("layer_norm_eps", 1e-5)
        kw.setdefault("patch_size", 32)
        super().__init__(**kw)


class ViTConfig(VisionConfig):
    model_type = "vit"

    def __init__(self, qkv_bias=True, **kw):
        kw.setdefault("hidden_act", "gelu")
        kw.setdefault("layer_norm_eps", 1e-12)
        self.qkv_bias = qkv_bias
        super().__init__(**kw)


def encoder_block(x, ln1, q, k, v, o, ln2, fc1, fc2, act: str, num_heads: int, mask: A.AttnMask, attn_impl=None,
                  scale: float | None = None):
    """Pre-LN transformer block shared by every encoder family (modules are passed in, names differ per family)."""
    B, S, H = x.shape
    D = q.weight.shape[0] // num_heads if num_heads else 0
    h = ln1(x)
    hin = q.input_hook(h)
    biases = [q.bias, k.bias, v.bias] if (q.bias is not None or k.bias is not None or v.bias is not None) else None
    qkv = multi_linear(hin, [q.weight, k.weight, v.weight], biases, tp=q.tp_spec(h))
    nh = q.weight.shape[0] // D
    qh = qkv[..., : nh * D].view(B, S, nh, D)
    kh = qkv[..., nh * D : 2 * nh * D].view(B, S, nh, D)
    vh = qkv[..., 2 * nh * D :].view(B, S, nh, D)
    if attn_impl is not None:
        a = attn_impl(qh, kh, vh, mask, scale)
    else:
        a = A.attention(qh, kh, vh, mask, scale)
    a = o(a.reshape(B, S, nh * D))
    h2, x = ln2(a, x)  # x <- x + a ; h2 = LN(x)
    m = fc2(E.activation(fc1(h2), act))
    return x + m


class _MLP(nn.Module):
    def __init__(self, hidden, inter, names=("fc1", "fc2")):
        super().__init__()
        setattr(self, names[0], cnn.Linear(hidden, inter))
        setattr(self, names[1], cnn.Linear(inter, hidden))


class _SelfAttn(nn.Module):
    def __init__(self, hidden, num_heads, bias=True, k_bias=True):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = hidden // num_heads
        self.q_proj = cnn.Linear(hidden, hidden, bias=bias)
        self.k_proj = cnn.Linear(hidden, hidden, bias=bias and k_bias)
        self.v_proj = cnn.Linear(hidden, hidden, bias=bias)
        self.out_proj = cnn.Linear(hidden, hidden, bias=bias)
        self.attn_impl = None


class SiglipEncoderLayer(nn.Module):
    """HF names: ``layer_norm1``, ``self_attn.{q,k,v,out}_proj``, ``layer_norm2``, ``mlp.fc1/fc2``."""

    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.act = config.hidden_act
        self.self_attn = _SelfAttn(H, config.num_attention_heads)
        self.layer_norm1 = cnn.LayerNorm(H, config.layer_norm_eps)
        self.mlp = _MLP(H, config.intermediate_size)
        self.layer_norm2 = cnn.LayerNorm(H, config.layer_norm_eps)

    def forward(self, x, mask):
        a = self.self_attn
        return encoder_block(x, self.layer_norm1, a.q_proj, a.k_proj, a.v_proj, a.out_proj, self.layer_norm2,
                             self.mlp.fc1, self.mlp.fc2, self.act, a.num_heads, mask, a.attn_impl)


class _Encoder(nn.Module):
    def __init__(self, config, layer_cls, list_name="layers"):
        super().__init__()
        self.list_name = list_name
        setattr(self, list_name, nn.ModuleList([layer_cls(config) for _ in range(config.num_hidden_layers)]))

    def run(self, x, mask, ckpt: bool):
        for layer in getattr(self, self.list_name):
            if is_released(layer):
                continue
            if ckpt and torch.is_grad_enabled():
                x = checkpoint_layer(layer, x, mask)
            else:
                x = layer(x, mask)
        return x


class SiglipVisionEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.patch_size = config.patch_size
        self.patch_embedding = nn.Conv2d(config.num_channels, config.hidden_size, config.patch_size, config.patch_size)
        self.num_patches = (config.image_size // config.patch_size) ** 2
        self.position_embedding = nn.Embedding(self.num_patches, config.hidden_size)

    def forward(self, pixel_values):
        x = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype))
        x = x.flatten(2).transpose(1, 2)
        return x + self.position_embedding.weight[: x.shape[1]].unsqueeze(0)


class SiglipPoolingHead(nn.Module):
    """Attention-pooling head (``vision_model.head``): a learned probe attends over the patch tokens."""

    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.probe = nn.Parameter(torch.randn(1, 1, H) * 0.02)
        self.attention = nn.MultiheadAttention(H, config.num_attention_heads, batch_first=True)
        self.layernorm = cnn.LayerNorm(H, config.layer_norm_eps)
        self.mlp = _MLP(H, config.intermediate_size)
        self.act = config.hidden_act

    def forward(self, x):
        probe = self.probe.expand(x.shape[0], -1, -1).to(x.dtype)
        h = self.attention(probe, x, x, need_weights=False)[0]
        r = h
        h = self.layernorm(h)
        h = r + self.mlp.fc2(E.activation(self.mlp.fc1(h), self.act))
        return h[:, 0]


class _SiglipVisionTransformer(nn.Module):
    def __init__(self, config, with_head=True):
        super().__init__()
        self.embeddings = SiglipVisionEmbeddings(config)
        self.encoder = _Encoder(config, SiglipEncoderLayer)
        self.post_layernorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.head = SiglipPoolingHead(config) if with_head else None


class _VisionBase(PreTrainedModel):
    main_input_name = "pixel_values"

    def _stage_input(self, pixel_values, hidden_states, embed_name, embed_fn):
        if hidden_states is not None:
            return hidden_states
        assert self.holds(embed_name), "this stage has no embeddings: pass hidden_states"
        x = embed_fn(pixel_values)
        group = getattr(self, "_cp_group", None)
        if group is not None:
            from ..parallel import comm

            x = comm.split_forward_gather_backward(x, 1, group)  # contiguous uniform token chunks
        return x

    def _attn_mask(self, device):
        """Full attention; under context parallelism the mask carries the gather state."""
        group = getattr(self, "_cp_group", None)
        if group is None:
            return A.AttnMask.full()
        from ..parallel.cp import ContextParallelState

        return ContextParallelState(group, None, None, device).local_mask


class SiglipVisionModel(_VisionBase):
    config_class = SiglipVisionConfig

    def __init__(self, config):
        super().__init__(config)
        self.vision_model = _SiglipVisionTransformer(config, getattr(config, "vision_use_head", True))

    @classmethod
    def module_names(cls, config):
        names = ["vision_model.embeddings"]
        names += [f"vision_model.encoder.layers.{i}" for i in range(config.num_hidden_layers)]
        names += ["vision_model.post_layernorm", "vision_model.head"]
        return names

    def forward(self, pixel_values=None, hidden_states=None, output_hidden_states=False, **kw):
        vm = self.vision_model
        x = self._stage_input(pixel_values, hidden_states, "vision_model.embeddings", lambda p: vm.embeddings(p))
        x = vm.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if not self.holds("vision_model.post_layernorm"):
            return ModelOutput(hidden_states=x)
        last = vm.post_layernorm(x)
        pooled = vm.head(last) if (vm.head is not None and not is_released(vm.head)) else None
        return ModelOutput(last_hidden_state=last, pooler_output=pooled)


# ------------------------------------------------------------------------------------------------ CLIP
class CLIPEncoderLayer(SiglipEncoderLayer):
    pass


class CLIPVisionEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.class_embedding = nn.Parameter(torch.randn(H) * 0.02)
        self.patch_embedding = nn.Conv2d(config.num_channels, H, config.patch_size, config.patch_size, bias=False)
        self.num_positions = (config.image_size // config.patch_size) ** 2 + 1
        self.position_embedding = nn.Embedding(self.num_positions, H)

    def forward(self, pixel_values):
        x = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        cls = self.class_embedding.expand(x.shape[0], 1, -1).to(x.dtype)
        x = torch.cat([cls, x], dim=1)
        return x + self.position_embedding.weight[: x.shape[1]].unsqueeze(0)


class _CLIPVisionTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embeddings = CLIPVisionEmbeddings(config)
        self.pre_layrnorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)  # (sic) HF spelling
        self.encoder = _Encoder(config, CLIPEncoderLayer)
        self.post_layernorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)


class CLIPVisionModel(_VisionBase):
    config_class = CLIPVisionConfig

    def __init__(self, config):
        super().__init__(config)
        self.vision_model = _CLIPVisionTransformer(config)

    @classmethod
    def module_names(cls, config):
        names = ["vision_model.embeddings", "vision_model.pre_layrnorm"]
        names += [f"vision_model.encoder.layers.{i}" for i in range(config.num_hidden_layers)]
        names += ["vision_model.post_layernorm"]
        return names

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        vm = self.vision_model
        x = self._stage_input(pixel_values, hidden_states, "vision_model.embeddings",
                              lambda p: vm.pre_layrnorm(vm.embeddings(p)))
        x = vm.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if not self.holds("vision_model.post_layernorm"):
            return ModelOutput(hidden_states=x)
        pooled = vm.post_layernorm(x[:, 0])
        return ModelOutput(last_hidden_state=x, pooler_output=pooled)


# ------------------------------------------------------------------------------------------------ ViT
class _ViTSelfAttention(nn.Module):
    def __init__(self, H, bias):
        super().__init__()
        self.query = cnn.Linear(H, H, bias=bias)
        self.key = cnn.Linear(H, H, bias=bias)
        self.value = cnn.Linear(H, H, bias=bias)


class _ViTDense(nn.Module):
    def __init__(self, i, o):
        super().__init__()
        self.dense = cnn.Linear(i, o)


class _ViTAttention(nn.Module):
    def __init__(self, H, bias):
        super().__init__()
        self.attention = _ViTSelfAttention(H, bias)
        self.output = _ViTDense(H, H)


class ViTLayer(nn.Module):
    """HF names: ``attention.attention.{query,key,value}``, ``attention.output.dense``, ``intermediate.dense``,
    ``output.dense``, ``layernorm_before``, ``layernorm_after``."""

    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.act = config.hidden_act
        self.attention = _ViTAttention(H, getattr(config, "qkv_bias", True))
        self.intermediate = _ViTDense(H, config.intermediate_size)
        self.output = _ViTDense(config.intermediate_size, H)
        self.layernorm_before = cnn.LayerNorm(H, config.layer_norm_eps)
        self.layernorm_after = cnn.LayerNorm(H, config.layer_norm_eps)
        self.attn_impl = None

    def forward(self, x, mask):
        a = self.attention.attention
        return encoder_block(x, self.layernorm_before, a.query, a.key, a.value, self.attention.output.dense,
                             self.layernorm_after, self.intermediate.dense, self.output.dense, self.act, self.num_heads,
                             mask, self.attn_impl)


class _ViTPatchEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.projection = nn.Conv2d(config.num_channels, config.hidden_size, config.patch_size, config.patch_size)


class ViTEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        n = (config.image_size // config.patch_size) ** 2
        self.cls_token = nn.Parameter(torch.randn(1, 1, H) * 0.02)
        self.patch_embeddings = _ViTPatchEmbeddings(config)
        self.position_embeddings = nn.Parameter(torch.randn(1, n + 1, H) * 0.02)

    def forward(self, pixel_values):
        w = self.patch_embeddings.projection.weight
        x = self.patch_embeddings.projection(pixel_values.to(w.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        return x + self.position_embeddings[:, : x.shape[1]].to(x.dtype)


class _ViTPooler(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = cnn.Linear(config.hidden_size, config.hidden_size)

    def forward(self, x):
        return torch.tanh(self.dense(x[:, 0]))


class ViTModel(_VisionBase):
    config_class = ViTConfig

    def __init__(self, config, add_pooling_layer=True):
        super().__init__(config)
        self.embeddings = ViTEmbeddings(config)
        self.encoder = _Encoder(config, ViTLayer, "layer")
        self.layernorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.pooler = _ViTPooler(config) if add_pooling_layer else None

    @classmethod
    def module_names(cls, config):
        return ["embeddings"] + [f"encoder.layer.{i}" for i in range(config.num_hidden_layers)] + ["layernorm", "pooler"]

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        x = self._stage_input(pixel_values, hidden_states, "embeddings", lambda p: self.embeddings(p))
        x = self.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if not self.holds("layernorm"):
            return ModelOutput(hidden_states=x)
        last = self.layernorm(x)
        pooled = self.pooler(last) if (self.pooler is not None and not is_released(self.pooler)) else None
        return ModelOutput(last_hidden_state=last, pooler_output=pooled)


register_model("siglip_vision_model", SiglipVisionConfig, SiglipVisionModel)
register_model("clip_vision_model", CLIPVisionConfig, CLIPVisionModel)
register_model("vit", ViTConfig, ViTModel)
