"""Build a :class:`MultimodalModel` from a composite Hugging Face checkpoint (LLaVA-NeXT, Qwen2-VL).

The reference does this in ``MultimodalModel.from_pretrained_multimodal_model`` with the adapter classes
``LlavaNextModel`` / ``Qwen2VLModel`` (cornstarch/models/multimodal_language_model/modeling_multimodal_language_model.py:45-327,
:752-772): the composite model is cut into vision tower, projector and language model, and callbacks reproduce the
glue the composite forward had (feature-layer selection, dropping the CLS token, the Qwen2-VL merger as projector).

Here the cut happens on the state dict, so nothing of ``transformers`` has to be instantiated:

    model = from_pretrained_multimodal_model("path/to/llava-next-checkpoint")          # a local directory
    model = multimodal_from_state_dict("llava_next", config_dict, state_dict)          # or tensors already in memory

LLaVA-NeXT: ``vision_feature_layer = -k`` is honoured by building the CLIP tower without its last ``k - 1`` layers;
the multi-resolution ("anyres") packing with ``image_newline`` is not reproduced - every image contributes the patch
tokens of its base resolution, the layout :class:`MultimodalProcessor` produces for a CLIP encoder.
"""

from __future__ import annotations

import json
import os
from collections import OrderedDict

import torch
import torch.nn as nn

from ..checkpoint.io import load_state_dict_any
from ..models import llama as L
from ..models import vision as V
from ..models import vision_extra as X
from ..models.base import registered
from .modeling import ModalEncoderModule, MultimodalModel, MultimodalProjector, MultimodalProjectorConfig


def _strip(sd: dict, prefix: str) -> dict:
    return OrderedDict((k[len(prefix):], v) for k, v in sd.items() if k.startswith(prefix))


def _norm_composite_keys(sd: dict) -> dict:
    """Keys of a composite checkpoint without the optional leading ``model.``: releases of ``transformers`` differ in where
    they put it (``model.language_model...`` next to ``language_model.lm_head.weight`` in one and the same file)."""
    return OrderedDict((k[len("model."):] if k.startswith("model.") else k, v) for k, v in sd.items())


def _language_model_part(body: dict) -> dict:
    """``language_model.*`` (and a top-level ``lm_head.*``) -> the state dict of a causal LM (``model.*`` + ``lm_head.*``)."""
    llm = OrderedDict()
    for k, v in body.items():
        if k.startswith("lm_head."):
            llm[k] = v
        elif k.startswith("language_model.lm_head."):
            llm[k[len("language_model."):]] = v
        elif k.startswith("language_model.model."):
            llm[k[len("language_model."):]] = v
        elif k.startswith("language_model."):
            llm["model." + k[len("language_model."):]] = v
    return llm


def split_llava_next_state_dict(sd: dict) -> dict[str, dict]:
    """Keys of ``LlavaNextForConditionalGeneration`` (any of the layouts ``transformers`` has written) -> per-module state dicts."""
    body = _norm_composite_keys(sd)
    vision = _strip(body, "vision_tower.")
    proj = _strip(body, "multi_modal_projector.")
    llm = _language_model_part(body)
    projector = OrderedDict()
    for name, new in (("linear_1", "in_proj"), ("linear_2", "out_proj")):
        for p in ("weight", "bias"):
            if f"{name}.{p}" in proj:
                projector[f"projection.{new}.{p}"] = proj[f"{name}.{p}"]
    extras = {k: v for k, v in body.items() if k == "image_newline"}
    return {"vision": vision, "projector": projector, "language_model": llm, "extras": extras}


def split_qwen2_vl_state_dict(sd: dict) -> dict[str, dict]:
    body = _norm_composite_keys(sd)
    visual = _strip(body, "visual.")
    merger = OrderedDict((k, v) for k, v in visual.items() if k.startswith("merger."))
    vision = OrderedDict((k, v) for k, v in visual.items() if not k.startswith("merger."))
    llm = _language_model_part(body)
    if not any(k.startswith("model.") for k in llm):
        # oldest layout: the decoder's tensors sit directly under ``model.`` next to ``model.visual.``
        llm = OrderedDict((k, v) for k, v in sd.items() if k.startswith("model.") and not k.startswith("model.visual."))
        if "lm_head.weight" in sd:
            llm["lm_head.weight"] = sd["lm_head.weight"]
    projector = OrderedDict(("projection." + k[len("merger."):], v) for k, v in merger.items())
    return {"vision": vision, "projector": projector, "language_model": llm, "extras": {}}


def _drop_cls(inputs, output):
    h = output["last_hidden_state"] if isinstance(output, dict) else output[0]
    return (h[:, 1:],)


def _text_model(text_cfg: dict):
    mt = text_cfg.get("model_type", "llama")
    reg = registered(mt)
    assert reg is not None, f"no language model registered for model_type '{mt}'"
    cfg_cls, model_cls = reg
    return model_cls(cfg_cls.from_dict(text_cfg))


class _PassThroughMerger(nn.Module):
    """Stands where the Qwen2-VL merger was: the merger itself becomes the projector."""

    def forward(self, x):
        return x


def multimodal_from_state_dict(model_type: str, config: dict, state_dict: dict, dtype=None, device=None) -> MultimodalModel:
    if model_type in ("llava_next", "llava"):
        # LLaVA-1.5 has the modules and key names of LLaVA-NeXT without ``image_newline``; every image is one base tile
        parts = split_llava_next_state_dict(state_dict)
        vcfg = dict(config["vision_config"])
        layer = config.get("vision_feature_layer", -2)
        assert isinstance(layer, int) and layer < 0, "a single negative vision_feature_layer is supported"
        keep = vcfg["num_hidden_layers"] + layer + 1  # -1 keeps all layers, -2 drops the last one, ...
        vcfg["num_hidden_layers"] = keep
        tower = vcfg.pop("model_type", None) or "clip_vision_model"
        vkw = {k: v for k, v in vcfg.items() if k in (
            "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_channels", "image_size",
            "patch_size", "hidden_act", "layer_norm_eps")}
        if tower.startswith("siglip"):
            vision = V.SiglipVisionModel(V.SiglipVisionConfig(**vkw, vision_use_head=False))
        else:
            vision = V.CLIPVisionModel(V.CLIPVisionConfig(**vkw))
        vsd = {k: v for k, v in parts["vision"].items() if not _layer_index_at_least(k, keep)}
        if tower.startswith("siglip"):
            # the feature layer's output is taken before SigLIP's final LayerNorm and pooling head
            vision.hold_only([n for n in vision.module_names(vision.config) if n not in ("vision_model.post_layernorm", "vision_model.head")])
            vsd = {k: v for k, v in vsd.items() if not k.startswith(("vision_model.post_layernorm.", "vision_model.head."))}
        llm = _text_model(config["text_config"])
        pc = MultimodalProjectorConfig(encoder_config=vision.config, text_config=llm.config, projection_type="mlp",
                                       activation=config.get("projector_hidden_act", "gelu"))
        projector = MultimodalProjector(pc)
        strategy = config.get("vision_feature_select_strategy", "default")
        enc = ModalEncoderModule(vision, projector, postprocess_module_callback=_drop_cls if strategy == "default" else None or _keep_all)
        token_id = config.get("image_token_index", config.get("image_token_id"))
    elif model_type == "qwen2_vl":
        parts = split_qwen2_vl_state_dict(state_dict)
        vc = {k: v for k, v in config["vision_config"].items() if k in (
            "depth", "embed_dim", "hidden_size", "hidden_act", "mlp_ratio", "num_heads", "in_channels", "patch_size",
            "spatial_merge_size", "temporal_patch_size")}
        vision = X.Qwen2VisionTransformerPretrainedModel(X.Qwen2VLVisionConfig(**vc))
        merger = vision.merger
        vision.merger = _PassThroughMerger()
        # the tower now ends at the transformer blocks: its width (what the projector check compares) is embed_dim
        import copy

        vision.config = copy.copy(vision.config)
        vision.config.out_hidden_size = vision.config.hidden_size
        vision.config.hidden_size = vc["embed_dim"]
        text_cfg = dict(config.get("text_config") or {k: v for k, v in config.items() if k != "vision_config"})
        text_cfg["model_type"] = "qwen2"
        llm = _text_model(text_cfg)
        pc = MultimodalProjectorConfig(in_features=vc["embed_dim"], out_features=llm.config.hidden_size, projection_type="mlp",
                                       encoder_model_type="qwen2_vl", language_model_type="qwen2")
        projector = MultimodalProjector(pc, projection=merger)
        vsd = parts["vision"]
        enc = ModalEncoderModule(vision, projector, additional_args=["grid_thw"])
        token_id = config.get("image_token_id", config.get("image_token_index"))
    else:
        raise NotImplementedError(f"from_pretrained_multimodal_model supports llava, llava_next and qwen2_vl, not '{model_type}'")

    _load(vision, vsd, "vision tower")
    _load(projector, parts["projector"], "projector")
    _load(llm, parts["language_model"], "language model")
    model = MultimodalModel(encoders={"vision": enc}, language_model=llm)
    if token_id is not None:
        model.set_modality_token_ids({"vision": int(token_id)})
    model.extras = parts["extras"]
    if dtype is not None or device is not None:
        model = model.to(device=device, dtype=dtype)
    return model


def _keep_all(inputs, output):
    if isinstance(output, dict):
        h = output["last_hidden_state"] if "last_hidden_state" in output else output["hidden_states"]
    else:
        h = output[0]
    return (h,)


def _layer_index_at_least(key: str, n: int) -> bool:
    marker = "encoder.layers."
    if marker not in key:
        return False
    idx = int(key.split(marker, 1)[1].split(".", 1)[0])
    return idx >= n


def _load(module, sd, what: str):
    missing, unexpected = module.load_state_dict(sd, strict=False)
    missing = [m for m in missing if "rotary" not in m]
    if missing or unexpected:
        raise RuntimeError(f"{what}: missing keys {missing[:5]}..., unexpected keys {list(unexpected)[:5]}...")


def from_pretrained_multimodal_model(path: str, dtype=None, device=None) -> MultimodalModel:
    """``path``: a local checkpoint directory of a composite HF model (``config.json`` + safetensors / bin shards)."""
    with open(os.path.join(path, "config.json")) as f:
        config = json.load(f)
    return multimodal_from_state_dict(config["model_type"], config, load_state_dict_any(path), dtype=dtype, device=device)
