"""EvaCLIP: text tower, the joint two-tower model and the ``*WithProjection`` variants, with the checkpoint parameter
names of the reference's EvaCLIP implementation.

The vision tower lives in :mod:`.vision_extra` (``EvaCLIPVisionModel``); this module adds what the reference defines in
cornstarch/models/evaclip/modeling_evaclip.py: the text embeddings (:170-207), ``EvaCLIPTextTransformer`` /
``EvaCLIPTextModel`` (:674-809), ``EvaCLIPModel`` (:904-1096) and ``EvaCLIPTextModelWithProjection`` /
``EvaCLIPVisionModelWithProjection`` (:1098-1206), plus the configurations of configuration_evaclip.py:17-454.

Both towers share one encoder layer (``EvaCLIPEncoderLayer``: pre-norm or post-norm, LayerNorm or RMSNorm, optional
q/k/v biases) on the shared kernels: fused q|k|v GEMM, flash attention (causal for text, full for images), fused norms
and activations.  The text tower's causal mask plus an optional padding mask is a bitfield mask (padding tokens carry no
bits), so padded batches stay on the attention kernel.

One deliberate difference: the reference stores ``logit_scale = tensor(100.0)`` and multiplies the similarity by
``logit_scale.exp()`` (e^100); here ``logit_scale`` holds ``log(100)`` (or ``logit_scale_init_value`` when the
configuration gives one), so the similarity is scaled by 100, CLIP's cap.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import nn as cnn
from ..ops import attention as A
from .base import ModelOutput, PretrainedConfig, PreTrainedModel, register_model
from .vision import _Encoder
from .vision_extra import EvaCLIPEncoderLayer, EvaCLIPVisionConfig, EvaCLIPVisionModel, _eva_norm, _EvaVisionTransformer

_TEXT_BITS = (1 << 62) | 1


class EvaCLIPTextConfig(PretrainedConfig):
    model_type = "evaclip_text_model"
    composite_key = "text_config"

    def __init__(self, vocab_size=49408, hidden_size=512, intermediate_size=2048, projection_dim=512, num_hidden_layers=12,
                 num_attention_heads=8, max_position_embeddings=77, hidden_act="gelu", layer_norm_eps=1e-5,
                 attention_dropout=0.0, initializer_range=0.02, initializer_factor=1.0, q_bias=True, k_bias=True, v_bias=True,
                 post_layernorm=False, pad_token_id=1, bos_token_id=0, eos_token_id=2, use_rms_norm=False, **kw):
        self.vocab_size, self.hidden_size, self.intermediate_size = vocab_size, hidden_size, intermediate_size
        self.projection_dim, self.num_hidden_layers, self.num_attention_heads = projection_dim, num_hidden_layers, num_attention_heads
        self.max_position_embeddings, self.hidden_act, self.layer_norm_eps = max_position_embeddings, hidden_act, layer_norm_eps
        self.attention_dropout, self.initializer_range, self.initializer_factor = attention_dropout, initializer_range, initializer_factor
        self.q_bias, self.k_bias, self.v_bias, self.post_layernorm = q_bias, k_bias, v_bias, post_layernorm
        self.pad_token_id, self.bos_token_id, self.eos_token_id, self.use_rms_norm = pad_token_id, bos_token_id, eos_token_id, use_rms_norm
        super().__init__(**kw)


class EvaCLIPConfig(PretrainedConfig):
    """Both towers: ``text_config`` / ``vision_config`` as configuration objects or plain dicts."""

    model_type = "evaclip"

    def __init__(self, text_config=None, vision_config=None, projection_dim=512, logit_scale_init_value=None, **kw):
        def build(c, cls):
            if c is None:
                return cls()
            if isinstance(c, dict):
                return cls.from_dict(c)
            return c

        self.text_config = build(text_config, EvaCLIPTextConfig)
        self.vision_config = build(vision_config, EvaCLIPVisionConfig)
        self.projection_dim = projection_dim
        self.logit_scale_init_value = logit_scale_init_value
        super().__init__(**kw)

    @classmethod
    def from_text_vision_configs(cls, text_config: EvaCLIPTextConfig, vision_config: EvaCLIPVisionConfig, **kw):
        return cls(text_config=text_config.to_dict(), vision_config=vision_config.to_dict(), **kw)


class EvaCLIPTextEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.token_embedding = nn.Embedding(config.vocab_size, config.hidden_size)
        self.position_embedding = nn.Embedding(config.max_position_embeddings, config.hidden_size)

    def forward(self, input_ids=None, position_ids=None, inputs_embeds=None):
        x = self.token_embedding(input_ids) if inputs_embeds is None else inputs_embeds
        S = x.shape[-2]
        pos = self.position_embedding.weight[:S].unsqueeze(0) if position_ids is None else self.position_embedding(position_ids)
        return x + pos.to(x.dtype)


class _EvaTextTransformer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embeddings = EvaCLIPTextEmbeddings(config)
        self.encoder = _Encoder(config, EvaCLIPEncoderLayer)
        self.final_layer_norm = _eva_norm(config)


def _text_mask(attention_mask) -> A.AttnMask:
    """Causal attention; with a padding mask (1 = real token) padded tokens neither attend nor are attended to."""
    if attention_mask is None:
        return A.AttnMask.causal()
    keep = attention_mask.bool()
    bits = torch.where(keep, torch.full_like(keep, _TEXT_BITS, dtype=torch.int64), torch.zeros_like(keep, dtype=torch.int64))
    return A.AttnMask.bitfield(bits)


class EvaCLIPTextModel(PreTrainedModel):
    """``text_model.*``: token + position embeddings, causal encoder, final norm; pooled output = the hidden state at the
    end-of-text token (the highest token id of each sequence)."""

    config_class = EvaCLIPTextConfig
    main_input_name = "input_ids"

    def __init__(self, config):
        super().__init__(config)
        self.text_model = _EvaTextTransformer(config)

    @classmethod
    def module_names(cls, config):
        return (["text_model.embeddings"] + [f"text_model.encoder.layers.{i}" for i in range(config.num_hidden_layers)]
                + ["text_model.final_layer_norm"])

    def get_input_embeddings(self):
        return self.text_model.embeddings.token_embedding

    def set_input_embeddings(self, value):
        self.text_model.embeddings.token_embedding = value

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, hidden_states=None, **kw):
        if input_ids is None and hidden_states is None:
            raise ValueError("You have to specify input_ids")
        tm = self.text_model
        if hidden_states is None:
            assert self.holds("text_model.embeddings"), "this stage has no embeddings: pass hidden_states"
            input_ids = input_ids.view(-1, input_ids.shape[-1])
            x = tm.embeddings(input_ids=input_ids, position_ids=position_ids)
        else:
            x = hidden_states
        x = tm.encoder.run(x, _text_mask(attention_mask), self.gradient_checkpointing and self.training)
        if not self.holds("text_model.final_layer_norm"):
            return ModelOutput(hidden_states=x)
        last = tm.final_layer_norm(x)
        pooled = None
        if input_ids is not None:
            eot = input_ids.to(last.device).argmax(dim=-1)
            pooled = last[torch.arange(last.shape[0], device=last.device), eot]
        return ModelOutput(last_hidden_state=last, pooler_output=pooled)


class EvaCLIPTextModelWithProjection(EvaCLIPTextModel):
    """Text tower + ``text_projection`` (no bias): ``text_embeds`` are the projected pooled outputs."""

    def __init__(self, config):
        super().__init__(config)
        self.text_projection = cnn.Linear(config.hidden_size, config.projection_dim, bias=False)

    @classmethod
    def module_names(cls, config):
        return super().module_names(config) + ["text_projection"]

    def forward(self, input_ids=None, attention_mask=None, position_ids=None, **kw):
        out = super().forward(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids, **kw)
        if "pooler_output" not in out or not self.holds("text_projection"):
            return out
        return ModelOutput(text_embeds=self.text_projection(out.pooler_output), last_hidden_state=out.last_hidden_state)


class EvaCLIPVisionModelWithProjection(EvaCLIPVisionModel):
    """Vision tower + ``visual_projection`` (no bias): ``image_embeds`` are the projected class-token outputs."""

    def __init__(self, config):
        super().__init__(config)
        self.visual_projection = cnn.Linear(config.hidden_size, config.projection_dim, bias=False)

    @classmethod
    def module_names(cls, config):
        return super().module_names(config) + ["visual_projection"]

    def get_input_embeddings(self):
        return self.vision_model.embeddings.patch_embedding

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        out = super().forward(pixel_values=pixel_values, hidden_states=hidden_states, **kw)
        if "pooler_output" not in out or not self.holds("visual_projection"):
            return out
        return ModelOutput(image_embeds=self.visual_projection(out.pooler_output), last_hidden_state=out.last_hidden_state)


def clip_loss(similarity: torch.Tensor) -> torch.Tensor:
    """Symmetric contrastive loss over a ``[texts, images]`` similarity matrix whose diagonal holds the matching pairs."""
    tgt = torch.arange(similarity.shape[0], device=similarity.device)
    ce = nn.functional.cross_entropy
    return (ce(similarity.float(), tgt) + ce(similarity.float().t(), tgt)) / 2.0


class EvaCLIPModel(PreTrainedModel):
    """Two towers with projections into a shared space; ``forward`` returns the scaled cosine similarities of every
    text / image pair (and the contrastive loss when ``return_loss``)."""

    config_class = EvaCLIPConfig

    def __init__(self, config):
        super().__init__(config)
        tc, vc = config.text_config, config.vision_config
        self.text_model = _EvaTextTransformer(tc)
        self.vision_model = _EvaVisionTransformer(vc)
        self.visual_projection = cnn.Linear(vc.hidden_size, config.projection_dim, bias=False)
        self.text_projection = cnn.Linear(tc.hidden_size, config.projection_dim, bias=False)
        init = config.logit_scale_init_value if config.logit_scale_init_value is not None else math.log(100.0)
        self.register_buffer("logit_scale", torch.tensor(float(init)), persistent=False)

    @classmethod
    def module_names(cls, config):
        t = ["text_model.embeddings"] + [f"text_model.encoder.layers.{i}" for i in range(config.text_config.num_hidden_layers)]
        v = ["vision_model.embeddings"] + [f"vision_model.encoder.layers.{i}" for i in range(config.vision_config.num_hidden_layers)]
        return t + ["text_model.final_layer_norm", "text_projection"] + v + ["vision_model.post_layernorm", "visual_projection"]

    def _text(self, input_ids, attention_mask=None, position_ids=None):
        tm = self.text_model
        input_ids = input_ids.view(-1, input_ids.shape[-1])
        x = tm.embeddings(input_ids=input_ids, position_ids=position_ids)
        x = tm.encoder.run(x, _text_mask(attention_mask), self.gradient_checkpointing and self.training)
        last = tm.final_layer_norm(x)
        pooled = last[torch.arange(last.shape[0], device=last.device), input_ids.to(last.device).argmax(dim=-1)]
        return ModelOutput(last_hidden_state=last, pooler_output=pooled)

    def _vision(self, pixel_values):
        vm = self.vision_model
        x = vm.encoder.run(vm.embeddings(pixel_values), A.AttnMask.full(), self.gradient_checkpointing and self.training)
        return ModelOutput(last_hidden_state=x, pooler_output=vm.post_layernorm(x[:, 0]))

    def encode_text(self, input_ids=None, attention_mask=None, position_ids=None, **kw):
        return self.text_projection(self._text(input_ids, attention_mask, position_ids).pooler_output)

    def encode_image(self, pixel_values=None, **kw):
        return self.visual_projection(self._vision(pixel_values).pooler_output)

    get_text_features = encode_text
    get_image_features = encode_image

    def forward(self, input_ids=None, pixel_values=None, attention_mask=None, position_ids=None, return_loss=False, **kw):
        vision_out = self._vision(pixel_values)
        text_out = self._text(input_ids, attention_mask, position_ids)
        image_embeds = self.visual_projection(vision_out.pooler_output).float()
        text_embeds = self.text_projection(text_out.pooler_output).float()
        image_embeds = image_embeds / image_embeds.norm(p=2, dim=-1, keepdim=True)
        text_embeds = text_embeds / text_embeds.norm(p=2, dim=-1, keepdim=True)
        logits_per_text = torch.matmul(text_embeds, image_embeds.t()) * self.logit_scale.exp()
        out = ModelOutput(logits_per_image=logits_per_text.t(), logits_per_text=logits_per_text, text_embeds=text_embeds,
                          image_embeds=image_embeds, text_model_output=text_out, vision_model_output=vision_out)
        if return_loss:
            out["loss"] = clip_loss(logits_per_text)
        return out


register_model("evaclip_text_model", EvaCLIPTextConfig, EvaCLIPTextModel)
register_model("evaclip", EvaCLIPConfig, EvaCLIPModel)

__all__ = ["EvaCLIPConfig", "EvaCLIPTextConfig", "EvaCLIPVisionConfig", "EvaCLIPModel", "EvaCLIPTextModel", "EvaCLIPVisionModel",
           "EvaCLIPTextModelWithProjection", "EvaCLIPVisionModelWithProjection", "EvaCLIPTextEmbeddings", "clip_loss"]
