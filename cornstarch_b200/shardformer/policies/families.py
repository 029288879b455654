"""Policy classes under the per-family names the reference uses (``LlamaForCausalLMPolicy``, ``MixtralModelPolicy``, ...;
cornstarch/shardformer/policies/<family>.py).  The decoder families share one implementation here: the differences between
them are in the model's spec, not in how it is sharded."""

from .multimodal import ModalModulePolicy  # noqa: F401
from .models import (  # noqa: F401
    BertForMultipleChoicePolicy,
    BertForNextSentencePredictionPolicy,
    BertForPreTrainingPolicy,
    BertForQuestionAnsweringPolicy,
    BertForSequenceClassificationPolicy,
    BertForTokenClassificationPolicy,
    BertLMHeadModelPolicy,
    DecoderForSequenceClassificationPolicy,
    Dinov2BackbonePolicy,
    Dinov2ForImageClassificationPolicy,
    GPT2DoubleHeadsModelPolicy,
    GPT2ForQuestionAnsweringPolicy,
    GPT2ForSequenceClassificationPolicy,
    GPT2ForTokenClassificationPolicy,
    OPTForQuestionAnsweringPolicy,
    OPTForSequenceClassificationPolicy,
    BertForMaskedLMPolicy,
    BertModelPolicy,
    CLIPVisionModelPolicy,
    DecoderForCausalLMPolicy,
    DecoderModelPolicy,
    Dinov2ModelPolicy,
    EvaCLIPVisionModelPolicy,
    GPT2LMHeadModelPolicy,
    GPT2ModelPolicy,
    InternVisionModelPolicy,
    Llama4ForCausalLMPolicy,
    Llama4TextModelPolicy,
    MoeForCausalLMPolicy,
    MultimodalProjectorPolicy,
    OPTForCausalLMPolicy,
    OPTModelPolicy,
    Phi4MultimodalAudioModelPolicy,
    PixtralVisionModelPolicy,
    Qwen2AudioEncoderPolicy,
    Qwen2VisionTransformerPolicy,
    SiglipVisionModelPolicy,
    ViTModelPolicy,
    WhisperEncoderPolicy,
)

for _family in ("Llama", "Mistral", "Qwen2", "Qwen3", "Gemma", "Gemma2", "Gemma3", "Phi3"):
    globals()[f"{_family}Policy"] = DecoderModelPolicy
    globals()[f"{_family}ModelPolicy"] = DecoderModelPolicy
    globals()[f"{_family}ForCausalLMPolicy"] = DecoderForCausalLMPolicy
for _family in ("Mixtral", "Qwen3Moe"):
    globals()[f"{_family}Policy"] = MoeForCausalLMPolicy
    globals()[f"{_family}ModelPolicy"] = MoeForCausalLMPolicy
    globals()[f"{_family}ForCausalLMPolicy"] = MoeForCausalLMPolicy
Llama4Policy = Llama4TextModelPolicy
SiglipVisionTransformerPolicy = SiglipVisionModelPolicy
CLIPVisionTransformerPolicy = CLIPVisionModelPolicy
GPT2Policy = GPT2ModelPolicy
BertPolicy = BertModelPolicy
OPTPolicy = OPTModelPolicy
Phi4MultimodalAudioPolicy = Phi4MultimodalAudioModelPolicy
LlamaForSequenceClassificationPolicy = DecoderForSequenceClassificationPolicy
