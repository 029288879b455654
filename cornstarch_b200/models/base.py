"""Model base classes: HF-style configs, ``save_pretrained`` / ``from_pretrained``, pipeline hooks.

Models in this package are written from scratch with HF-compatible parameter names and
``config.json`` fields, so a checkpoint directory produced here (``config.json`` +
``model.safetensors`` or sharded safetensors + ``model.safetensors.index.json``) has the layout the
reference produces through HF ``PreTrainedModel`` (tests/test_utils/test_pretrained_projection.py:75-80
in the reference).  Instead of patching HF forwards per policy (cornstarch/shardformer/modeling/*.py),
each model natively understands pipeline stages: :meth:`PreTrainedModel.module_names` lists the
pipeline-assignable units in order (the reference's ``get_all_modules``) and
:meth:`PreTrainedModel.hold_only` drops everything a stage does not own.
"""

from __future__ import annotations

import copy
import json
import os
from typing import Any

import torch
import torch.nn as nn

CONFIG_NAME = "config.json"
WEIGHTS_NAME = "model.safetensors"
WEIGHTS_INDEX_NAME = "model.safetensors.index.json"

_MODEL_REGISTRY: dict[str, tuple[type, type]] = {}


def register_model(model_type: str, config_cls: type, model_cls: type) -> None:
    """``AutoConfig`` / ``AutoModel`` style registration keyed by ``model_type``."""
    _MODEL_REGISTRY[model_type] = (config_cls, model_cls)


def registered(model_type: str):
    return _MODEL_REGISTRY.get(model_type)


_CHECKPOINT_PREFIXES = ("", "model.", "encoder.", "model.encoder.", "vision_tower.", "model.vision_tower.", "visual.",
                        "model.visual.", "audio_tower.", "model.audio_tower.", "language_model.", "model.language_model.",
                        "transformer.", "bert.", "vit.", "dinov2.", "model.decoder.")


def _strip_checkpoint_prefix(sd: dict, wanted: set) -> dict:
    """A sub-model is often loaded from the checkpoint of a larger one (the Whisper encoder from a full Whisper model, a
    vision tower from a vision-language model): find the key prefix under which most of the wanted tensors live and
    return that part of the state dict without it (the counterpart of ``base_model_prefix`` handling in ``transformers``)."""
    best, best_hits = "", sum(k in sd for k in wanted)
    for p in _CHECKPOINT_PREFIXES[1:]:
        hits = sum((p + k) in sd for k in wanted)
        if hits > best_hits:
            best, best_hits = p, hits
    if not best:
        return sd
    out = {k[len(best):]: v for k, v in sd.items() if k.startswith(best)}
    for k in wanted - set(out):
        # a checkpoint may keep a few tensors elsewhere (``language_model.lm_head.weight`` next to ``model.language_model.*``)
        for p in _CHECKPOINT_PREFIXES:
            if (p + k) in sd:
                out[k] = sd[p + k]
                break
    return out


class PretrainedConfig:
    """Attribute bag with HF ``config.json`` round-tripping.  Subclasses set ``model_type`` and defaults."""

    model_type: str = ""

    def __init__(self, **kwargs):
        for k, v in kwargs.items():
            setattr(self, k, v)

    def to_dict(self) -> dict[str, Any]:
        out = {}
        for k, v in self.__dict__.items():
            if k.startswith("_"):
                continue
            if isinstance(v, PretrainedConfig):
                v = v.to_dict()
            elif isinstance(v, torch.dtype):
                v = str(v).replace("torch.", "")
            out[k] = v
        out["model_type"] = self.model_type
        return out

    @classmethod
    def from_dict(cls, d: dict[str, Any]):
        d = dict(d)
        d.pop("model_type", None)
        return cls(**d)

    @classmethod
    def from_hf(cls, hf_config):
        """Build from a ``transformers`` config object (or anything with ``to_dict``)."""
        d = hf_config.to_dict() if hasattr(hf_config, "to_dict") else dict(hf_config)
        return cls.from_dict(d)

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, CONFIG_NAME), "w") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)

    @classmethod
    def from_pretrained(cls, path: str):
        with open(os.path.join(path, CONFIG_NAME)) as f:
            d = json.load(f)
        if cls is PretrainedConfig:
            reg = registered(d.get("model_type", ""))
            if reg is not None:
                return reg[0].from_dict(d)
        sub = getattr(cls, "composite_key", None)
        if sub and isinstance(d.get(sub), dict):
            d = d[sub]  # the config of a composite model (CLIP / SigLIP with both towers, a vision-language model)
        return cls.from_dict(d)

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict()})"

    def __eq__(self, other):
        return isinstance(other, PretrainedConfig) and self.to_dict() == other.to_dict()


class PreTrainedModel(nn.Module):
    """Common behaviour of every model: config, (de)serialisation, pipeline-stage pruning."""

    config_class = PretrainedConfig
    # names of sub-modules that can be placed on a pipeline stage, produced by `module_names(config)`
    supports_gradient_checkpointing = True

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.gradient_checkpointing = False
        self._held: set[str] | None = None  # None = everything

    # ---- pipeline -------------------------------------------------------------------------
    @classmethod
    def module_names(cls, config) -> list[str]:
        """Ordered names of the pipeline-assignable units (``PipelineTemplate.get_modules``)."""
        raise NotImplementedError

    def holds(self, name: str) -> bool:
        return self._held is None or name in self._held

    def hold_only(self, names: list[str]) -> None:
        """Release every pipeline unit that is not in ``names``: its parameters are freed, the module itself is kept on
        the meta device inside the placeholder.  A unit in ``names`` that an earlier call released comes back from there
        with meta parameters, to be materialised (``materialize_meta``) and filled from a checkpoint - what re-planning
        the pipelines of a running job needs."""
        all_names = self.module_names(self.config)
        unknown = set(names) - set(all_names)
        assert not unknown, f"unknown module names {sorted(unknown)}"
        self._held = set(names)
        for n in all_names:
            parent, attr = self._resolve_parent(n)
            if parent is None:
                continue
            in_list = isinstance(parent, (nn.ModuleList, nn.Sequential))
            target = parent[int(attr)] if in_list else getattr(parent, attr)

            def put(m):
                if in_list:
                    parent[int(attr)] = m
                else:
                    setattr(parent, attr, m)

            if n in self._held:
                if isinstance(target, _Released) and target.stash is not None:
                    put(target.stash)
                continue
            if isinstance(target, _Released):
                continue
            if isinstance(target, nn.Module) and not any(True for _ in target.parameters()):
                continue  # stateless helpers (rotary tables, activations, poolers) cost nothing to keep
            put(_Released(target.to("meta") if isinstance(target, nn.Module) else None))

    def _resolve_parent(self, dotted: str):
        obj = self
        parts = dotted.split(".")
        for p in parts[:-1]:
            if not hasattr(obj, p) and not (isinstance(obj, (nn.ModuleList, nn.Sequential)) and p.isdigit()):
                return None, None
            obj = obj[int(p)] if p.isdigit() else getattr(obj, p)
        last = parts[-1]
        if isinstance(obj, (nn.ModuleList, nn.Sequential)) and last.isdigit():
            return obj, last
        return (obj, last) if hasattr(obj, last) else (None, None)

    # ---- checkpointing of activations -----------------------------------------------------------
    def gradient_checkpointing_enable(self, gradient_checkpointing_kwargs: dict | None = None):
        """``gradient_checkpointing_kwargs={"keep_last_layers": k}``: the last ``k`` decoder layers this rank holds keep
        their activations (no recomputation) - for when memory is left over; other keys (``use_reentrant``) are accepted
        and ignored."""
        keep = int((gradient_checkpointing_kwargs or {}).get("keep_last_layers", 0))
        self.gradient_checkpointing = True
        self.recompute_keep_layers = keep
        for m in self.modules():
            if m is not self and isinstance(m, PreTrainedModel):
                m.gradient_checkpointing = True
                m.recompute_keep_layers = keep

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False
        for m in self.modules():
            if m is not self and isinstance(m, PreTrainedModel):
                m.gradient_checkpointing = False

    def resize_token_embeddings(self, new_num_tokens: int):
        """Grow (or shrink) the input embedding table and, when present, the output head to ``new_num_tokens`` rows; new
        rows start at the mean of the existing ones.  Tied tables stay tied.  Returns the input embedding module."""
        emb = self.get_input_embeddings()
        head = self.get_output_embeddings() if hasattr(self, "get_output_embeddings") else None
        tied = head is not None and head.weight is emb.weight

        def grown(w: torch.Tensor) -> nn.Parameter:
            new = w.new_empty(new_num_tokens, w.shape[1])
            n = min(w.shape[0], new_num_tokens)
            new[:n] = w.data[:n]
            if new_num_tokens > n:
                new[n:] = w.data.float().mean(0, keepdim=True).to(w.dtype)
            return nn.Parameter(new, requires_grad=w.requires_grad)

        if emb.weight.shape[0] != new_num_tokens:
            emb.weight = grown(emb.weight)
            if hasattr(emb, "num_embeddings"):
                emb.num_embeddings = new_num_tokens
            if head is not None:
                head.weight = emb.weight if tied else grown(head.weight)
                if hasattr(head, "out_features"):
                    head.out_features = new_num_tokens
            if hasattr(self.config, "vocab_size"):
                self.config.vocab_size = new_num_tokens
        return emb

    # ---- (de)serialisation ---------------------------------------------------------------------
    def save_pretrained(self, path: str, max_shard_size: int | None = None, safe_serialization: bool = True):
        from ..checkpoint.io import save_state_dict_sharded

        os.makedirs(path, exist_ok=True)
        self.config.save_pretrained(path)
        sd = {k: v.detach().cpu().contiguous() for k, v in self.state_dict().items()}
        save_state_dict_sharded(sd, path, max_shard_size=max_shard_size, use_safetensors=safe_serialization)

    @classmethod
    def from_pretrained(cls, path: str, config=None, dtype=None, device=None, strict: bool = True, **kwargs):
        from ..checkpoint.io import load_state_dict_any

        if config is None:
            # several families share one model class (the decoder): the checkpoint's ``model_type`` picks the config
            # class, and with it the family's details (q/k norms, fused projections, biases, experts)
            with open(os.path.join(path, CONFIG_NAME)) as f:
                reg = registered(json.load(f).get("model_type", ""))
            if reg is not None and (issubclass(reg[1], cls) or issubclass(cls, reg[1])):
                config = reg[0].from_pretrained(path)
                if issubclass(reg[1], cls):
                    cls = reg[1]  # e.g. the MoE subclass for a Mixtral checkpoint
            else:
                config = cls.config_class.from_pretrained(path)
        model = cls(config, **kwargs)
        sd = _strip_checkpoint_prefix(load_state_dict_any(path), set(model.state_dict().keys()))
        missing, unexpected = model.load_state_dict(sd, strict=False)
        if getattr(config, "tie_word_embeddings", False):
            # tied output embeddings are stored once: the head shares the input embedding's tensor
            missing = [k for k in missing if not k.endswith("lm_head.weight") and "decoder.weight" not in k]
        if strict and missing:
            raise RuntimeError(f"from_pretrained: missing={missing} unexpected={list(unexpected)[:8]}")
        if unexpected:
            # tensors of other parts of a larger checkpoint (a text tower, a decoder): ignored, as ``transformers`` does
            import logging

            logging.getLogger(__name__).info("from_pretrained(%s): %d tensors of the checkpoint are not used", path, len(unexpected))
        if dtype is not None or device is not None:
            model = model.to(device=device, dtype=dtype)
        return model

    @property
    def device(self):
        try:
            return next(self.parameters()).device
        except StopIteration:
            return torch.device("cpu")

    @property
    def dtype(self):
        try:
            return next(self.parameters()).dtype
        except StopIteration:
            return torch.float32

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())


class _Released(nn.Module):
    """Placeholder left where a pipeline unit was released; calling it is a bug in the stage plan.  The released module
    itself (parameters on the meta device: shapes and dtypes, no storage) waits in ``stash`` for a later re-plan."""

    def __init__(self, stash: nn.Module | None = None):
        super().__init__()
        object.__setattr__(self, "stash", stash)  # not a sub-module: invisible to parameters() and state_dict()

    def forward(self, *a, **k):
        raise RuntimeError("this module is not held by the current pipeline stage")


def is_released(m) -> bool:
    return isinstance(m, _Released)


class ModelOutput(dict):
    """Dict with attribute access (``out.loss``, ``out["logits"]``), the shape HF models return."""

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v


def clone_config(config):
    return copy.deepcopy(config)
