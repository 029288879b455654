"""``MultimodalProcessor``: per-modality processors + a tokenizer, with modality placeholders expanded.

Inputs are given per modality (``encoder_inputs={"vision": {"images": ...}, "audio": {"raw_speech": ...}}``,
``llm_inputs={"text": ...}``).  Each modality processor runs on its own inputs; the number of features
every item will produce is computed by a per-modality function (defaults exist for the common HF
processor classes); every occurrence of the modality token in the text is expanded to that many copies;
the text is tokenized; the result is one dict whose FIRST key is ``input_ids``.  On construction the
modality tokens are registered as special tokens and their ids are handed to the model
(``model.set_modality_token_ids``).  Behaviour follows the reference class
(cornstarch/models/multimodal_language_model/processing_multimodal_language_model.py:22-314).
"""

from __future__ import annotations

import copy
import functools
import inspect
import logging
import math
from typing import Any, Callable

logger = logging.getLogger(__name__)


def num_features_audio_static(inputs: dict, outputs: dict, config) -> list[int]:
    return [config.max_source_positions] * outputs["input_features"].shape[0]


def num_features_vision_clip(inputs: dict, outputs: dict, config) -> list[int]:
    return [(config.image_size // config.patch_size) ** 2 + 1] * outputs["pixel_values"].shape[0]


def num_features_vision_static(inputs: dict, outputs: dict, config) -> list[int]:
    return [(config.image_size // config.patch_size) ** 2] * outputs["pixel_values"].shape[0]


def num_features_pixtral(inputs: dict, outputs: dict, config) -> list[int]:
    ps = config.patch_size if isinstance(config.patch_size, (tuple, list)) else (config.patch_size, config.patch_size)
    out = []
    for h, w in outputs["image_sizes"]:
        out.append(int(math.ceil(h / ps[0]) * math.ceil(w / ps[1])))
    return out


def num_features_qwen2vl(inputs: dict, outputs: dict, config) -> list[int] | None:
    grid = outputs.get("image_grid_thw", None)
    if grid is None:
        return None
    merge = config.spatial_merge_size ** 2
    return [int(grid[i].prod()) // merge for i in range(len(grid))]


def num_features_phi4audio(inputs: dict, outputs: dict, config) -> list[int]:
    feats = outputs["audio_input_features"]
    return [math.ceil(feats.shape[1] / config.time_reduction)] * feats.shape[0]


processor_type_to_num_feature_calculation_func = {
    "ViTImageProcessor": num_features_vision_static,
    "CLIPImageProcessor": num_features_vision_clip,
    "SiglipImageProcessor": num_features_vision_static,
    "BitImageProcessor": num_features_vision_static,
    "PixtralImageProcessor": num_features_pixtral,
    "Qwen2VLImageProcessor": num_features_qwen2vl,
    "WhisperFeatureExtractor": num_features_audio_static,
    "Phi4MultimodalFeatureExtractor": num_features_phi4audio,
}
# the "Fast" variants of HF image processors behave the same
for _k in list(processor_type_to_num_feature_calculation_func):
    processor_type_to_num_feature_calculation_func[_k + "Fast"] = processor_type_to_num_feature_calculation_func[_k]

_PLACEHOLDER = "<|placeholder|>"


class BatchFeature(dict):
    """Ordered dict with attribute access and ``.to(device)`` (the shape of HF's ``BatchFeature``)."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def to(self, *args, **kwargs):
        return BatchFeature({k: (v.to(*args, **kwargs) if hasattr(v, "to") else v) for k, v in self.items()})


class MultimodalProcessor:
    def __init__(self, encoder_processors: dict[str, Any], llm_tokenizer, model,
                 num_feature_calculation_funcs: dict[str, Callable] | None = None,
                 predefined_tokens: dict[str, str] | None = None):
        funcs = dict(num_feature_calculation_funcs or {})
        for key, proc in encoder_processors.items():
            if key in funcs:
                continue
            default = processor_type_to_num_feature_calculation_func.get(type(proc).__name__)
            if default is not None:
                funcs[key] = functools.partial(default, config=model.encoders[key].module.config)
            else:
                logger.warning("num_feature_calculation_func for %s is not provided.", key)
        self.encoder_processors = encoder_processors
        self.llm_tokenizer = llm_tokenizer
        self.num_feature_calculation_funcs = funcs
        self.tokens: dict[str, str] = {}
        self._set_modality_tokens(model, predefined_tokens or {})

    def _set_modality_tokens(self, model, predefined_tokens: dict[str, str]) -> None:
        tokens = {k: predefined_tokens.get(k, f"<{k}>") for k in self.encoder_processors}
        self.llm_tokenizer.add_special_tokens({"additional_special_tokens": list(tokens.values())})
        ids = {k: self.llm_tokenizer.convert_tokens_to_ids(t) for k, t in tokens.items()}
        model.set_modality_token_ids(ids, len(self.llm_tokenizer))
        self.tokens = tokens

    def __call__(self, encoder_inputs: dict[str, dict] | None = None, llm_inputs: dict | None = None,
                 return_tensors: str = "pt", **kwargs) -> BatchFeature:
        encoder_inputs, llm_inputs = encoder_inputs or {}, llm_inputs or {}
        if "text" not in llm_inputs:
            raise ValueError("The llm_inputs should have a key 'text' for the text input.")
        text = copy.deepcopy(llm_inputs["text"])
        if not isinstance(text, list):
            text = [text]
        result: dict = {}
        for key, enc_in in encoder_inputs.items():
            if key not in self.num_feature_calculation_funcs:
                raise ValueError(f"num_feature_calculation_funcs for {key} is not defined.")
            if key not in self.tokens:
                raise ValueError(f"tokens for {key} is not defined.")
            proc = self.encoder_processors[key]
            accepted = list(inspect.signature(proc.__call__).parameters.keys())
            proc_in = {k: v for k, v in kwargs.items() if k in accepted}
            proc_in.update(enc_in)
            out = proc(**proc_in, return_tensors=return_tensors)
            result.update(out)
            counts = self.num_feature_calculation_funcs[key](proc_in, out)
            if counts and isinstance(counts[0], list):
                counts = [c for per_batch in counts for c in per_batch]
            idx = 0
            tok = self.tokens[key]
            for i in range(len(text)):
                while tok in text[i]:
                    text[i] = text[i].replace(tok, _PLACEHOLDER * int(counts[idx]), 1)
                    idx += 1
                text[i] = text[i].replace(_PLACEHOLDER, tok)
        accepted = list(inspect.signature(self.llm_tokenizer.__call__).parameters.keys())
        tok_in = {k: v for k, v in kwargs.items() if k in accepted}
        tok_in.update(llm_inputs)
        tok_in["text"] = text
        text_out = self.llm_tokenizer(**tok_in, return_tensors=return_tensors)
        result.update(text_out)
        input_ids = result.pop("input_ids")
        return BatchFeature({"input_ids": input_ids, **result})  # input_ids first: batch size is read from the first key

    def batch_decode(self, *a, **k):
        return self.llm_tokenizer.batch_decode(*a, **k)

    def decode(self, *a, **k):
        return self.llm_tokenizer.decode(*a, **k)

    def apply_chat_template(self, *a, **k):
        return self.llm_tokenizer.apply_chat_template(*a, **k)
