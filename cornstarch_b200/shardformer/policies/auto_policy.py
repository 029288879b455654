"""Fully-qualified model class name -> policy class (``get_autopolicy`` / ``get_policy_type`` / ``import_policy``).

Keys cover this package's model classes and, as aliases, the HF ``transformers`` class names the
reference registers (cornstarch/shardformer/policies/auto_policy.py:12-248), so a template written for
``transformers.models.llama.modeling_llama.LlamaForCausalLM`` resolves to the same pipeline units.
"""

from __future__ import annotations

from . import models as P
from .multimodal import ModalModulePolicy

# task-head classes whose policy is named <class>Policy, here and (as transformers.models.<family>.modeling_<family>.<class>)
# in the reference's registry
_HEADS = ("BertForPreTraining", "BertLMHeadModel", "BertForSequenceClassification", "BertForTokenClassification",
          "BertForNextSentencePrediction", "BertForMultipleChoice", "BertForQuestionAnswering", "GPT2DoubleHeadsModel",
          "GPT2ForQuestionAnswering", "GPT2ForTokenClassification", "GPT2ForSequenceClassification",
          "OPTForSequenceClassification", "OPTForQuestionAnswering")

_NATIVE = {
    "cornstarch_b200.models.llama.DecoderModel": P.DecoderModelPolicy,
    "cornstarch_b200.models.llama.DecoderForCausalLM": P.DecoderForCausalLMPolicy,
    "cornstarch_b200.models.moe.MoeForCausalLM": P.MoeForCausalLMPolicy,
    "cornstarch_b200.models.vision.SiglipVisionModel": P.SiglipVisionModelPolicy,
    "cornstarch_b200.models.vision.CLIPVisionModel": P.CLIPVisionModelPolicy,
    "cornstarch_b200.models.vision.ViTModel": P.ViTModelPolicy,
    "cornstarch_b200.models.whisper.WhisperEncoder": P.WhisperEncoderPolicy,
    "cornstarch_b200.models.whisper.Qwen2AudioEncoder": P.Qwen2AudioEncoderPolicy,
    "cornstarch_b200.multimodal.modeling.MultimodalProjector": P.MultimodalProjectorPolicy,
    "cornstarch_b200.models.vision_extra.Dinov2Model": P.Dinov2ModelPolicy,
    "cornstarch_b200.models.vision_extra.EvaCLIPVisionModel": P.EvaCLIPVisionModelPolicy,
    "cornstarch_b200.models.vision_extra.InternVisionModel": P.InternVisionModelPolicy,
    "cornstarch_b200.models.vision_extra.PixtralVisionModel": P.PixtralVisionModelPolicy,
    "cornstarch_b200.models.vision_extra.Qwen2VisionTransformerPretrainedModel": P.Qwen2VisionTransformerPolicy,
    "cornstarch_b200.models.llama4.Llama4TextModel": P.Llama4TextModelPolicy,
    "cornstarch_b200.models.llama4.Llama4ForCausalLM": P.Llama4ForCausalLMPolicy,
    "cornstarch_b200.models.phi4_audio.Phi4MultimodalAudioModel": P.Phi4MultimodalAudioModelPolicy,
    "cornstarch_b200.models.text_legacy.GPT2Model": P.GPT2ModelPolicy,
    "cornstarch_b200.models.text_legacy.GPT2LMHeadModel": P.GPT2LMHeadModelPolicy,
    "cornstarch_b200.models.text_legacy.BertModel": P.BertModelPolicy,
    "cornstarch_b200.models.text_legacy.BertForMaskedLM": P.BertForMaskedLMPolicy,
    "cornstarch_b200.models.text_legacy.OPTModel": P.OPTModelPolicy,
    "cornstarch_b200.models.text_legacy.OPTForCausalLM": P.OPTForCausalLMPolicy,
    "cornstarch_b200.multimodal.modeling.ModalEncoderModule": ModalModulePolicy,
    "cornstarch_b200.multimodal.modeling.ModalDecoderModule": ModalModulePolicy,
    "cornstarch_b200.models.task_heads.DecoderForSequenceClassification": P.DecoderForSequenceClassificationPolicy,
    "cornstarch_b200.models.task_heads.Dinov2Backbone": P.Dinov2BackbonePolicy,
    "cornstarch_b200.models.task_heads.Dinov2ForImageClassification": P.Dinov2ForImageClassificationPolicy,
    **{f"cornstarch_b200.models.task_heads.{n}": getattr(P, n + "Policy") for n in _HEADS},
}


def _hf(family: str, module: str, base: str, causal: str):
    pre = f"transformers.models.{family}.modeling_{module}."
    return {pre + base: P.DecoderModelPolicy, pre + causal: P.DecoderForCausalLMPolicy}


_HF_ALIASES = {}
for fam, base, causal in (("llama", "LlamaModel", "LlamaForCausalLM"), ("mistral", "MistralModel", "MistralForCausalLM"),
                          ("qwen2", "Qwen2Model", "Qwen2ForCausalLM"), ("qwen3", "Qwen3Model", "Qwen3ForCausalLM"),
                          ("gemma", "GemmaModel", "GemmaForCausalLM"), ("gemma2", "Gemma2Model", "Gemma2ForCausalLM"),
                          ("gemma3", "Gemma3TextModel", "Gemma3ForCausalLM"), ("phi3", "Phi3Model", "Phi3ForCausalLM")):
    _HF_ALIASES.update(_hf(fam, fam, base, causal))
_HF_ALIASES.update({
    "transformers.models.mixtral.modeling_mixtral.MixtralModel": P.DecoderModelPolicy,
    "transformers.models.mixtral.modeling_mixtral.MixtralForCausalLM": P.MoeForCausalLMPolicy,
    "transformers.models.qwen3_moe.modeling_qwen3_moe.Qwen3MoeModel": P.DecoderModelPolicy,
    "transformers.models.qwen3_moe.modeling_qwen3_moe.Qwen3MoeForCausalLM": P.MoeForCausalLMPolicy,
    "transformers.models.siglip.modeling_siglip.SiglipVisionModel": P.SiglipVisionModelPolicy,
    "transformers.models.clip.modeling_clip.CLIPVisionModel": P.CLIPVisionModelPolicy,
    "transformers.models.vit.modeling_vit.ViTModel": P.ViTModelPolicy,
    "transformers.models.whisper.modeling_whisper.WhisperEncoder": P.WhisperEncoderPolicy,
    "transformers.models.qwen2_audio.modeling_qwen2_audio.Qwen2AudioEncoder": P.Qwen2AudioEncoderPolicy,
    "cornstarch.models.multimodal_language_model.modeling_multimodal_language_model.MultimodalProjector": P.MultimodalProjectorPolicy,
    "transformers.models.dinov2.modeling_dinov2.Dinov2Model": P.Dinov2ModelPolicy,
    "cornstarch.models.evaclip.modeling_evaclip.EvaCLIPVisionModel": P.EvaCLIPVisionModelPolicy,
    "cornstarch.models.intern_vit.modeling_intern_vit.InternVisionModel": P.InternVisionModelPolicy,
    "transformers.models.pixtral.modeling_pixtral.PixtralVisionModel": P.PixtralVisionModelPolicy,
    "transformers.models.qwen2_vl.modeling_qwen2_vl.Qwen2VisionTransformerPretrainedModel": P.Qwen2VisionTransformerPolicy,
    "transformers.models.llama4.modeling_llama4.Llama4TextModel": P.Llama4TextModelPolicy,
    "transformers.models.llama4.modeling_llama4.Llama4ForCausalLM": P.Llama4ForCausalLMPolicy,
    "transformers.models.phi4_multimodal.modeling_phi4_multimodal.Phi4MultimodalAudioModel": P.Phi4MultimodalAudioModelPolicy,
    "transformers.models.gpt2.modeling_gpt2.GPT2Model": P.GPT2ModelPolicy,
    "transformers.models.gpt2.modeling_gpt2.GPT2LMHeadModel": P.GPT2LMHeadModelPolicy,
    "transformers.models.bert.modeling_bert.BertModel": P.BertModelPolicy,
    "transformers.models.bert.modeling_bert.BertForMaskedLM": P.BertForMaskedLMPolicy,
    "transformers.models.opt.modeling_opt.OPTModel": P.OPTModelPolicy,
    "transformers.models.opt.modeling_opt.OPTForCausalLM": P.OPTForCausalLMPolicy,
    **{f"transformers.models.{n[:4].lower().rstrip('f')}.modeling_{n[:4].lower().rstrip('f')}.{n}": getattr(P, n + "Policy") for n in _HEADS},
    "transformers.models.llama.modeling_llama.LlamaForSequenceClassification": P.DecoderForSequenceClassificationPolicy,
    "transformers.models.dinov2.modeling_dinov2.Dinov2Backbone": P.Dinov2BackbonePolicy,
    "transformers.models.dinov2.modeling_dinov2.Dinov2ForImageClassification": P.Dinov2ForImageClassificationPolicy,
    # the language model of Qwen2-VL is a Qwen2 decoder (the reference maps the class to its Qwen2 causal-LM policy)
    "transformers.models.qwen2_vl.modeling_qwen2_vl.Qwen2VLForConditionalGeneration": P.DecoderForCausalLMPolicy,
    "cornstarch.models.multimodal_language_model.modeling_multimodal_language_model.ModalEncoderModule": ModalModulePolicy,
    "cornstarch.models.multimodal_language_model.modeling_multimodal_language_model.ModalDecoderModule": ModalModulePolicy,
})

_POLICY_LIST = {**_NATIVE, **_HF_ALIASES}


def register_policy(fullname: str, policy_cls) -> None:
    _POLICY_LIST[fullname] = policy_cls


def import_policy(fullname: str):
    return get_policy_type(fullname)


def get_policy_type(fullname: str):
    pol = _POLICY_LIST.get(fullname)
    if pol is None:
        # subclasses of registered model classes (e.g. LlamaForCausalLM = DecoderForCausalLM) resolve by MRO
        raise NotImplementedError(f"Auto policy for {fullname} is not implemented. Supported: {sorted(_POLICY_LIST)}")
    return pol


def get_autopolicy(fullname: str):
    """Instance of the policy registered for the fully-qualified class name."""
    return get_policy_type(fullname)()


def policy_for_model(model):
    """Policy instance for a model object, walking its class MRO."""
    for klass in type(model).__mro__:
        name = f"{klass.__module__}.{klass.__qualname__}"
        if name in _POLICY_LIST:
            pol = _POLICY_LIST[name]()
            pol.set_model(model)
            return pol
    raise NotImplementedError(f"no policy for {type(model)}")
