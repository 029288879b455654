"""More vision encoders with their checkpoint parameter names: DINOv2, EvaCLIP, InternViT, Pixtral and the
Qwen2-VL vision tower.

The reference covers these families with one policy and one patched forward each
(cornstarch/shardformer/policies/{dinov2,evaclip,intern_vit,pixtral,qwen2_vision}.py and
cornstarch/shardformer/modeling/ of the same names) and ships the EvaCLIP and InternViT model code itself
(cornstarch/models/evaclip/modeling_evaclip.py:129-900, cornstarch/models/intern_vit/modeling_intern_vit.py:35-415).
Here every family is a small native module on the shared kernels (fused q|k|v GEMM, flash attention with a full
mask, fused norms, GLU / GELU kernels); ``module_names`` returns the pipeline units the reference's
``get_all_modules`` lists.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from .. import nn as cnn
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.linear import multi_linear
from .base import ModelOutput, PretrainedConfig, is_released, register_model
from .vision import VisionConfig, _Encoder, _VisionBase


def _attend(qkv: torch.Tensor, nh: int, D: int, mask, attn_impl=None):
    B, S, _ = qkv.shape
    q, k, v = (qkv[..., i * nh * D : (i + 1) * nh * D].view(B, S, nh, D) for i in range(3))
    fn = attn_impl or A.attention
    return fn(q, k, v, mask, None).reshape(B, S, nh * D)


# ------------------------------------------------------------------------------------------------ DINOv2
class Dinov2Config(VisionConfig):
    model_type = "dinov2"

    def __init__(self, mlp_ratio=4, qkv_bias=True, layerscale_value=1.0, use_swiglu_ffn=False, **kw):
        kw.setdefault("hidden_act", "gelu")
        kw.setdefault("layer_norm_eps", 1e-6)
        kw.setdefault("patch_size", 14)
        self.mlp_ratio, self.qkv_bias, self.layerscale_value, self.use_swiglu_ffn = mlp_ratio, qkv_bias, layerscale_value, use_swiglu_ffn
        super().__init__(**kw)
        self.intermediate_size = int(self.hidden_size * mlp_ratio)


class _LayerScale(nn.Module):
    def __init__(self, H, init):
        super().__init__()
        self.lambda1 = nn.Parameter(init * torch.ones(H))

    def forward(self, x):
        return x * self.lambda1.to(x.dtype)


class _DinoSelfAttention(nn.Module):
    def __init__(self, H, bias):
        super().__init__()
        self.query, self.key, self.value = cnn.Linear(H, H, bias=bias), cnn.Linear(H, H, bias=bias), cnn.Linear(H, H, bias=bias)


class _DinoDense(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.dense = cnn.Linear(H, H)


class _DinoAttention(nn.Module):
    def __init__(self, H, bias):
        super().__init__()
        self.attention = _DinoSelfAttention(H, bias)
        self.output = _DinoDense(H)


class _DinoMLP(nn.Module):
    def __init__(self, H, I):
        super().__init__()
        self.fc1, self.fc2 = cnn.Linear(H, I), cnn.Linear(I, H)


class _DinoSwiGLU(nn.Module):
    def __init__(self, H, I):
        super().__init__()
        hidden = (int(I * 2 / 3) + 7) // 8 * 8
        self.weights_in, self.weights_out = cnn.Linear(H, 2 * hidden), cnn.Linear(hidden, H)


class Dinov2Layer(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads, self.head_dim = config.num_attention_heads, H // config.num_attention_heads
        self.act, self.swiglu = config.hidden_act, config.use_swiglu_ffn
        self.norm1 = cnn.LayerNorm(H, config.layer_norm_eps)
        self.attention = _DinoAttention(H, config.qkv_bias)
        self.layer_scale1 = _LayerScale(H, config.layerscale_value)
        self.norm2 = cnn.LayerNorm(H, config.layer_norm_eps)
        self.mlp = _DinoSwiGLU(H, config.intermediate_size) if self.swiglu else _DinoMLP(H, config.intermediate_size)
        self.layer_scale2 = _LayerScale(H, config.layerscale_value)
        self.attn_impl = None

    def forward(self, x, mask):
        a = self.attention.attention
        biases = [a.query.bias, a.key.bias, a.value.bias] if a.query.bias is not None else None
        qkv = multi_linear(a.query.input_hook(self.norm1(x)), [a.query.weight, a.key.weight, a.value.weight], biases)
        o = self.attention.output.dense(_attend(qkv, self.num_heads, self.head_dim, mask, self.attn_impl))
        x = x + self.layer_scale1(o)
        h = self.norm2(x)
        if self.swiglu:
            m = self.mlp.weights_out(E.glu(self.mlp.weights_in(h), "silu"))
        else:
            m = self.mlp.fc2(E.activation(self.mlp.fc1(h), self.act))
        return x + self.layer_scale2(m)


class _DinoPatch(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.projection = nn.Conv2d(config.num_channels, config.hidden_size, config.patch_size, config.patch_size)


class Dinov2Embeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        n = (config.image_size // config.patch_size) ** 2
        self.cls_token = nn.Parameter(torch.randn(1, 1, H) * 0.02)
        self.mask_token = nn.Parameter(torch.zeros(1, H))
        self.patch_embeddings = _DinoPatch(config)
        self.position_embeddings = nn.Parameter(torch.randn(1, n + 1, H) * 0.02)

    def forward(self, pixel_values):
        w = self.patch_embeddings.projection.weight
        x = self.patch_embeddings.projection(pixel_values.to(w.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        return x + self.position_embeddings[:, : x.shape[1]].to(x.dtype)


class Dinov2Model(_VisionBase):
    config_class = Dinov2Config

    def __init__(self, config):
        super().__init__(config)
        self.embeddings = Dinov2Embeddings(config)
        self.encoder = _Encoder(config, Dinov2Layer, "layer")
        self.layernorm = cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)

    @classmethod
    def module_names(cls, config):
        return ["embeddings"] + [f"encoder.layer.{i}" for i in range(config.num_hidden_layers)] + ["layernorm"]

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        x = self._stage_input(pixel_values, hidden_states, "embeddings", lambda p: self.embeddings(p))
        x = self.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if not self.holds("layernorm"):
            return ModelOutput(hidden_states=x)
        last = self.layernorm(x)
        return ModelOutput(last_hidden_state=last, pooler_output=last[:, 0])


# ------------------------------------------------------------------------------------------------ EvaCLIP
class EvaCLIPVisionConfig(VisionConfig):
    model_type = "evaclip_vision_model"

    def __init__(self, use_rms_norm=False, q_bias=True, k_bias=True, v_bias=True, post_layernorm=False, projection_dim=512, **kw):
        kw.setdefault("hidden_act", "gelu")
        kw.setdefault("layer_norm_eps", 1e-5)
        kw.setdefault("patch_size", 14)
        self.use_rms_norm, self.q_bias, self.k_bias, self.v_bias = use_rms_norm, q_bias, k_bias, v_bias
        self.post_layernorm, self.projection_dim = post_layernorm, projection_dim
        super().__init__(**kw)


def _eva_norm(config):
    return cnn.RMSNorm(config.hidden_size, config.layer_norm_eps) if config.use_rms_norm else cnn.LayerNorm(config.hidden_size, config.layer_norm_eps)


class _EvaAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.k_proj = cnn.Linear(H, H, bias=config.k_bias)
        self.v_proj = cnn.Linear(H, H, bias=config.v_bias)
        self.q_proj = cnn.Linear(H, H, bias=config.q_bias)
        self.out_proj = cnn.Linear(H, H, bias=True)


class _EvaMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.fc1, self.fc2 = cnn.Linear(config.hidden_size, config.intermediate_size), cnn.Linear(config.intermediate_size, config.hidden_size)


class EvaCLIPEncoderLayer(nn.Module):
    """Pre-norm block, or (``post_layernorm``) the norm applied to each sub-layer's output before the residual add."""

    def __init__(self, config):
        super().__init__()
        self.num_heads, self.head_dim = config.num_attention_heads, config.hidden_size // config.num_attention_heads
        self.act, self.post = config.hidden_act, bool(config.post_layernorm)
        self.self_attn = _EvaAttention(config)
        self.layer_norm1 = _eva_norm(config)
        self.mlp = _EvaMLP(config)
        self.layer_norm2 = _eva_norm(config)
        self.attn_impl = None

    def _qkv(self, h):
        a = self.self_attn
        H = a.q_proj.weight.shape[0]
        zero = lambda: torch.zeros(H, dtype=h.dtype, device=h.device)  # noqa: E731
        bs = [a.q_proj.bias, a.k_proj.bias, a.v_proj.bias]
        biases = None if all(b is None for b in bs) else [b if b is not None else zero() for b in bs]
        return multi_linear(a.q_proj.input_hook(h), [a.q_proj.weight, a.k_proj.weight, a.v_proj.weight], biases)

    def forward(self, x, mask):
        h = x if self.post else self.layer_norm1(x)
        o = self.self_attn.out_proj(_attend(self._qkv(h), self.num_heads, self.head_dim, mask, self.attn_impl))
        x = x + (self.layer_norm1(o) if self.post else o)
        h = x if self.post else self.layer_norm2(x)
        m = self.mlp.fc2(E.activation(self.mlp.fc1(h), self.act))
        return x + (self.layer_norm2(m) if self.post else m)


class EvaCLIPVisionEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.class_embedding = nn.Parameter(torch.randn(H) * 0.02)
        self.patch_embedding = nn.Conv2d(config.num_channels, H, config.patch_size, config.patch_size, bias=True)
        self.position_embedding = nn.Embedding((config.image_size // config.patch_size) ** 2 + 1, H)

    def forward(self, pixel_values):
        x = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.expand(x.shape[0], 1, -1).to(x.dtype), x], dim=1)
        return x + self.position_embedding.weight[: x.shape[1]].unsqueeze(0)


class _EvaVisionTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embeddings = EvaCLIPVisionEmbeddings(config)
        self.encoder = _Encoder(config, EvaCLIPEncoderLayer)
        self.post_layernorm = _eva_norm(config)


class EvaCLIPVisionModel(_VisionBase):
    config_class = EvaCLIPVisionConfig

    def __init__(self, config):
        super().__init__(config)
        self.vision_model = _EvaVisionTransformer(config)

    @classmethod
    def module_names(cls, config):
        return (["vision_model.embeddings"] + [f"vision_model.encoder.layers.{i}" for i in range(config.num_hidden_layers)]
                + ["vision_model.post_layernorm"])

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        vm = self.vision_model
        x = self._stage_input(pixel_values, hidden_states, "vision_model.embeddings", lambda p: vm.embeddings(p))
        x = vm.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if not self.holds("vision_model.post_layernorm"):
            return ModelOutput(hidden_states=x)
        return ModelOutput(last_hidden_state=x, pooler_output=vm.post_layernorm(x[:, 0]))


# ------------------------------------------------------------------------------------------------ InternViT
class InternVisionConfig(VisionConfig):
    model_type = "intern_vit_6b"

    def __init__(self, qkv_bias=False, qk_normalization=True, initializer_factor=0.1, **kw):
        kw.setdefault("hidden_act", "gelu")
        kw.setdefault("layer_norm_eps", 1e-6)
        kw.setdefault("patch_size", 14)
        self.qkv_bias, self.qk_normalization, self.initializer_factor = qkv_bias, qk_normalization, initializer_factor
        super().__init__(**kw)


class _InternAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.qkv = cnn.Linear(H, 3 * H, bias=config.qkv_bias)
        self.qk_normalization = config.qk_normalization
        if self.qk_normalization:
            self.q_norm = cnn.RMSNorm(H, config.layer_norm_eps)
            self.k_norm = cnn.RMSNorm(H, config.layer_norm_eps)
        self.proj = cnn.Linear(H, H)


class _InternMLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.fc1, self.fc2 = cnn.Linear(config.hidden_size, config.intermediate_size), cnn.Linear(config.intermediate_size, config.hidden_size)


class InternVisionEncoderLayer(nn.Module):
    """``x += ls1 * attn(norm1(x)); x += ls2 * mlp(norm2(x))`` with a fused qkv projection and RMS-normalised q, k."""

    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads, self.head_dim, self.act = config.num_attention_heads, H // config.num_attention_heads, config.hidden_act
        self.attn = _InternAttention(config)
        self.mlp = _InternMLP(config)
        self.norm1 = cnn.RMSNorm(H, config.layer_norm_eps)
        self.norm2 = cnn.RMSNorm(H, config.layer_norm_eps)
        self.ls1 = nn.Parameter(config.initializer_factor * torch.ones(H))
        self.ls2 = nn.Parameter(config.initializer_factor * torch.ones(H))
        self.attn_impl = None

    def forward(self, x, mask):
        qkv = self.attn.qkv(self.norm1(x))
        if self.attn.qk_normalization:
            q, k, v = qkv.split(qkv.shape[-1] // 3, dim=-1)
            qkv = torch.cat([self.attn.q_norm(q.contiguous()), self.attn.k_norm(k.contiguous()), v], dim=-1)
        o = self.attn.proj(_attend(qkv, self.num_heads, self.head_dim, mask, self.attn_impl))
        x = x + o * self.ls1.to(x.dtype)
        m = self.mlp.fc2(E.activation(self.mlp.fc1(self.norm2(x)), self.act))
        return x + m * self.ls2.to(x.dtype)


class InternVisionEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        n = (config.image_size // config.patch_size) ** 2
        self.class_embedding = nn.Parameter(torch.randn(1, 1, H) * 0.02)
        self.patch_embedding = nn.Conv2d(config.num_channels, H, config.patch_size, config.patch_size)
        self.position_embedding = nn.Parameter(torch.randn(1, n + 1, H) * 0.02)

    def forward(self, pixel_values):
        x = self.patch_embedding(pixel_values.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_embedding.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        return x + self.position_embedding[:, : x.shape[1]].to(x.dtype)


class InternVisionModel(_VisionBase):
    config_class = InternVisionConfig

    def __init__(self, config):
        super().__init__(config)
        self.embeddings = InternVisionEmbeddings(config)
        self.encoder = _Encoder(config, InternVisionEncoderLayer)

    @classmethod
    def module_names(cls, config):
        return ["embeddings"] + [f"encoder.layers.{i}" for i in range(config.num_hidden_layers)]

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        x = self._stage_input(pixel_values, hidden_states, "embeddings", lambda p: self.embeddings(p))
        x = self.encoder.run(x, self._attn_mask(x.device), self.gradient_checkpointing and self.training)
        if is_released(self.encoder.layers[-1]):
            return ModelOutput(hidden_states=x)
        return ModelOutput(last_hidden_state=x, pooler_output=x[:, 0])


# ------------------------------------------------------------------------------------------------ Pixtral
class PixtralVisionConfig(VisionConfig):
    model_type = "pixtral"

    def __init__(self, head_dim=None, rope_theta=10000.0, **kw):
        kw.setdefault("hidden_act", "silu")
        kw.setdefault("hidden_size", 1024)
        kw.setdefault("intermediate_size", 4096)
        kw.setdefault("num_hidden_layers", 24)
        kw.setdefault("num_attention_heads", 16)
        kw.setdefault("image_size", 1024)
        kw.setdefault("patch_size", 16)
        kw.setdefault("layer_norm_eps", 1e-5)
        self.rope_theta = rope_theta
        super().__init__(**kw)
        self.head_dim = head_dim or self.hidden_size // self.num_attention_heads


class PixtralRotaryEmbedding(nn.Module):
    """2-D rotary tables: position ``h * side + w`` rotates half of the frequency pairs by ``h`` and half by ``w``."""

    def __init__(self, config):
        super().__init__()
        self.dim, self.theta = config.head_dim, config.rope_theta
        self.side = config.image_size // config.patch_size
        self._tables = None

    def tables(self, device):
        if self._tables is None or self._tables[0].device != torch.device(device):
            freqs = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=device) / self.dim))
            h = torch.arange(self.side, dtype=torch.float32, device=device)
            fh = torch.outer(h, freqs[::2])
            fw = torch.outer(h, freqs[1::2])
            ang = torch.cat([fh[:, None, :].expand(-1, self.side, -1), fw[None, :, :].expand(self.side, -1, -1)], dim=-1)
            ang = ang.reshape(self.side * self.side, self.dim // 2)
            self._tables = (ang.cos().contiguous(), ang.sin().contiguous())
        return self._tables


class _PixtralAttention(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.k_proj, self.v_proj = cnn.Linear(H, H, bias=False), cnn.Linear(H, H, bias=False)
        self.q_proj, self.o_proj = cnn.Linear(H, H, bias=False), cnn.Linear(H, H, bias=False)


class _PixtralMLP(nn.Module):
    def __init__(self, H, I):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = cnn.Linear(H, I, bias=False), cnn.Linear(H, I, bias=False), cnn.Linear(I, H, bias=False)


class PixtralAttentionLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.hidden_size
        self.num_heads, self.head_dim, self.act = config.num_attention_heads, config.head_dim, config.hidden_act
        self.attention_norm = cnn.RMSNorm(H, 1e-5)
        self.feed_forward = _PixtralMLP(H, config.intermediate_size)
        self.attention = _PixtralAttention(H)
        self.ffn_norm = cnn.RMSNorm(H, 1e-5)
        self.attn_impl = None

    def forward(self, x, mask, rope=None, pos=None):
        a, f = self.attention, self.feed_forward
        qkv = multi_linear(a.q_proj.input_hook(self.attention_norm(x)), [a.q_proj.weight, a.k_proj.weight, a.v_proj.weight])
        if rope is not None:
            qkv = E.rope_(qkv, rope[0], rope[1], pos, 2 * self.num_heads, self.head_dim)
        x = x + a.o_proj(_attend(qkv, self.num_heads, self.head_dim, mask, self.attn_impl))
        gu = multi_linear(f.gate_proj.input_hook(self.ffn_norm(x)), [f.gate_proj.weight, f.up_proj.weight])
        return x + f.down_proj(E.glu(gu, self.act))


class _PixtralTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layers = nn.ModuleList([PixtralAttentionLayer(config) for _ in range(config.num_hidden_layers)])


class PixtralVisionModel(_VisionBase):
    """Pixtral vision tower for a batch of equally sized images ``[B, 3, H, W]`` (each image is its own sequence)."""

    config_class = PixtralVisionConfig

    def __init__(self, config):
        super().__init__(config)
        self.patch_conv = nn.Conv2d(config.num_channels, config.hidden_size, config.patch_size, config.patch_size, bias=False)
        self.ln_pre = cnn.RMSNorm(config.hidden_size, 1e-5)
        self.patch_positional_embedding = PixtralRotaryEmbedding(config)
        self.transformer = _PixtralTransformer(config)

    @classmethod
    def module_names(cls, config):
        return ["patch_conv", "ln_pre", "patch_positional_embedding"] + [f"transformer.layers.{i}" for i in range(config.num_hidden_layers)]

    def forward(self, pixel_values=None, hidden_states=None, position_ids=None, **kw):
        from ..utils.recompute import checkpoint_layer

        if hidden_states is None:
            x = self.patch_conv(pixel_values.to(self.patch_conv.weight.dtype))
            B, H, gh, gw = x.shape
            x = self.ln_pre(x.flatten(2).transpose(1, 2))
            side = self.patch_positional_embedding.side
            hh, ww = torch.meshgrid(torch.arange(gh, device=x.device), torch.arange(gw, device=x.device), indexing="ij")
            position_ids = (hh * side + ww).reshape(1, -1).expand(B, -1).int().contiguous()
            group = getattr(self, "_cp_group", None)
            if group is not None:
                # context parallelism: contiguous token chunks per rank, and with them their 2-D rotary positions
                import torch.distributed as dist

                from ..parallel import comm

                x = comm.split_forward_gather_backward(x, 1, group)
                position_ids = torch.tensor_split(position_ids, dist.get_world_size(group), dim=1)[dist.get_rank(group)].contiguous()
        else:
            x = hidden_states
        rope = self.patch_positional_embedding.tables(x.device)
        mask = self._attn_mask(x.device)
        for layer in self.transformer.layers:
            if is_released(layer):
                continue
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint_layer(layer, x, mask, rope, position_ids)
            else:
                x = layer(x, mask, rope, position_ids)
        if is_released(self.transformer.layers[-1]):
            return ModelOutput(hidden_states=x, position_ids=position_ids)
        return ModelOutput(last_hidden_state=x)


# ------------------------------------------------------------------------------------------------ Qwen2-VL vision
class Qwen2VLVisionConfig(PretrainedConfig):
    model_type = "qwen2_vl"
    composite_key = "vision_config"

    def __init__(self, depth=32, embed_dim=1280, hidden_size=3584, hidden_act="quick_gelu", mlp_ratio=4, num_heads=16,
                 in_channels=3, patch_size=14, spatial_merge_size=2, temporal_patch_size=2, **kw):
        self.depth, self.embed_dim, self.hidden_size, self.hidden_act = depth, embed_dim, hidden_size, hidden_act
        self.mlp_ratio, self.num_heads, self.in_channels, self.patch_size = mlp_ratio, num_heads, in_channels, patch_size
        self.spatial_merge_size, self.temporal_patch_size = spatial_merge_size, temporal_patch_size
        super().__init__(**kw)

    num_hidden_layers = property(lambda self: self.depth)


class _QwenPatchEmbed(nn.Module):
    def __init__(self, config):
        super().__init__()
        k = (config.temporal_patch_size, config.patch_size, config.patch_size)
        self.shape = (config.in_channels, *k)
        self.proj = nn.Conv3d(config.in_channels, config.embed_dim, kernel_size=k, stride=k, bias=False)

    def forward(self, x):
        # x: [T, C * tp * ps * ps] flattened patches -> a plain GEMM with the reshaped conv kernel
        w = self.proj.weight.view(self.proj.weight.shape[0], -1)
        return cnn.linear(x.to(w.dtype), w)


class _QwenVisionAttention(nn.Module):
    def __init__(self, H):
        super().__init__()
        self.qkv, self.proj = cnn.Linear(H, 3 * H), cnn.Linear(H, H)


class _QwenVisionMLP(nn.Module):
    def __init__(self, H, I):
        super().__init__()
        self.fc1, self.fc2 = cnn.Linear(H, I), cnn.Linear(I, H)


class Qwen2VLVisionBlock(nn.Module):
    def __init__(self, config):
        super().__init__()
        H = config.embed_dim
        self.num_heads, self.head_dim, self.act = config.num_heads, H // config.num_heads, config.hidden_act
        self.norm1, self.norm2 = cnn.LayerNorm(H, 1e-6), cnn.LayerNorm(H, 1e-6)
        self.attn = _QwenVisionAttention(H)
        self.mlp = _QwenVisionMLP(H, int(H * config.mlp_ratio))
        self.attn_impl = None

    def forward(self, x, mask, rope, pos):
        qkv = E.rope_(self.attn.qkv(self.norm1(x)), rope[0], rope[1], pos, 2 * self.num_heads, self.head_dim)
        x = x + self.attn.proj(_attend(qkv, self.num_heads, self.head_dim, mask, self.attn_impl))
        return x + self.mlp.fc2(E.activation(self.mlp.fc1(self.norm2(x)), self.act))


class _QwenPatchMerger(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.width = config.embed_dim * config.spatial_merge_size ** 2
        self.ln_q = cnn.LayerNorm(config.embed_dim, 1e-6)
        self.mlp = nn.Sequential(cnn.Linear(self.width, self.width), nn.GELU(), cnn.Linear(self.width, config.hidden_size))

    def forward(self, x):
        h = self.ln_q(x)
        if h.dim() == 3:  # [images, tokens, C] (context parallelism keeps the image dimension): merge inside each image
            return self.mlp(h.reshape(h.shape[0], -1, self.width))
        return self.mlp(h.reshape(-1, self.width))


class _QwenVisionRotary(nn.Module):
    def __init__(self, dim, theta=10000.0):
        super().__init__()
        self.dim, self.theta = dim, theta

    def forward(self, n, device):
        inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=device) / self.dim))
        return torch.outer(torch.arange(n, dtype=torch.float32, device=device), inv)


class Qwen2VisionTransformerPretrainedModel(_VisionBase):
    """Qwen2-VL vision tower.  ``hidden_states`` (alias ``pixel_values``) are flattened patches ``[T, C*tp*ps*ps]`` and
    ``grid_thw`` gives each image's patch grid.  All images of a call must share one grid so that the batch is a dense
    ``[images, tokens]`` block with full attention per image (the reference enforces equal lengths the same way,
    cornstarch/shardformer/modeling/qwen2_vision.py:223-244)."""

    config_class = Qwen2VLVisionConfig
    main_input_name = "hidden_states"

    def __init__(self, config):
        super().__init__(config)
        self.spatial_merge_size = config.spatial_merge_size
        self.patch_embed = _QwenPatchEmbed(config)
        self.rotary_pos_emb = _QwenVisionRotary(config.embed_dim // config.num_heads // 2)
        self.blocks = nn.ModuleList([Qwen2VLVisionBlock(config) for _ in range(config.depth)])
        self.merger = _QwenPatchMerger(config)

    @classmethod
    def module_names(cls, config):
        return ["patch_embed", "rotary_pos_emb"] + [f"blocks.{i}" for i in range(config.depth)] + ["merger"]

    def rot_angles(self, grid_thw):
        m = self.spatial_merge_size
        out = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h).unsqueeze(1).expand(-1, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(w).unsqueeze(0).expand(h, -1).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).flatten()
            out.append(torch.stack([hp, wp], dim=-1).repeat(t, 1))
        pos = torch.cat(out, dim=0).to(grid_thw.device)
        table = self.rotary_pos_emb(int(grid_thw[:, 1:].max()), grid_thw.device)
        return table[pos].flatten(1)  # [T, head_dim/2]: h angles then w angles

    def forward(self, hidden_states=None, grid_thw=None, pixel_values=None, embedded=None, **kw):
        from ..utils.recompute import checkpoint_layer

        x = hidden_states if hidden_states is not None else pixel_values
        if embedded is None:
            x = self.patch_embed(x)
        n_img = grid_thw.shape[0]
        per = int(grid_thw[0].prod())
        assert bool((grid_thw.prod(-1) == per).all()), "all images of a call must have the same patch grid"
        ang = self.rot_angles(grid_thw)
        rope = (ang.cos().contiguous(), ang.sin().contiguous())
        pos = torch.arange(n_img * per, device=x.device, dtype=torch.int32).view(n_img, per)
        group = getattr(self, "_cp_group", None)
        if group is not None:
            # Context parallelism: every image's tokens are split over the ranks in whole merge groups (2 x 2 patches
            # are consecutive tokens), so that the merger can work on a rank's own tokens.  The image dimension is kept
            # in the output, [images, local tokens / merge, hidden], for the sequence gather that follows the projector.
            import torch.distributed as dist

            from ..parallel import comm

            ws, r = dist.get_world_size(group), dist.get_rank(group)
            unit = self.spatial_merge_size ** 2
            bounds = torch.tensor_split(torch.arange(per // unit), ws)[r]
            lo, hi = (int(bounds[0]) * unit, (int(bounds[-1]) + 1) * unit) if bounds.numel() else (0, 0)
            pos = pos[:, lo:hi].contiguous()
            if embedded is None:
                x = x.view(n_img, per // unit, -1)
                x = comm.split_forward_gather_backward(x, 1, group)
            per = hi - lo
        x = x.reshape(n_img, per, -1)
        mask = self._attn_mask(x.device)
        for blk in self.blocks:
            if is_released(blk):
                continue
            if self.gradient_checkpointing and self.training and torch.is_grad_enabled():
                x = checkpoint_layer(blk, x, mask, rope, pos)
            else:
                x = blk(x, mask, rope, pos)
        if is_released(self.merger):
            return ModelOutput(hidden_states=x.reshape(n_img * per, -1), embedded=True)
        if group is not None:
            return ModelOutput(last_hidden_state=self.merger(x))  # [images, local tokens / merge, hidden]
        return ModelOutput(last_hidden_state=self.merger(x.reshape(n_img * per, -1)))


register_model("dinov2", Dinov2Config, Dinov2Model)
register_model("evaclip_vision_model", EvaCLIPVisionConfig, EvaCLIPVisionModel)
register_model("intern_vit_6b", InternVisionConfig, InternVisionModel)
register_model("pixtral", PixtralVisionConfig, PixtralVisionModel)
register_model("qwen2_vl", Qwen2VLVisionConfig, Qwen2VisionTransformerPretrainedModel)
