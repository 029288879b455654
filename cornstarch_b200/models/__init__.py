"""Model families with Hugging Face parameter names: ``llama`` (Llama, Mistral, Qwen2/3, Gemma 1-3, Phi3), ``moe`` (Mixtral,
Qwen3-MoE), ``llama4``, ``text_legacy`` (GPT-2, BERT, OPT), ``vision`` (SigLIP, CLIP, ViT), ``vision_extra`` (DINOv2, EvaCLIP vision,
InternViT, Pixtral, Qwen2-VL vision), ``evaclip`` (EvaCLIP text tower and joint model), ``whisper`` (Whisper, Qwen2-Audio encoders), ``phi4_audio``.  Every module registers its
classes by ``model_type`` (the reference registers EvaCLIP and InternViT with the HF Auto classes,
cornstarch/models/__init__.py:1-15); :class:`AutoModel` looks a checkpoint's ``model_type`` up there."""

_FAMILY_MODULES = ("llama", "moe", "llama4", "text_legacy", "vision", "vision_extra", "evaclip", "whisper", "phi4_audio")


class AutoModel:
    """``AutoModel.from_pretrained(dir)``: the model class registered for the checkpoint's ``model_type``."""

    @staticmethod
    def from_pretrained(path: str, **kwargs):
        import importlib
        import json
        import os

        from .base import registered

        for name in _FAMILY_MODULES:  # importing a family module registers its model types
            importlib.import_module(f"{__name__}.{name}")
        with open(os.path.join(path, "config.json")) as f:
            model_type = json.load(f).get("model_type", "")
        reg = registered(model_type)
        if reg is None:
            raise ValueError(f"no model registered for model_type '{model_type}'")
        return reg[1].from_pretrained(path, **kwargs)


AutoModelForCausalLM = AutoModel
