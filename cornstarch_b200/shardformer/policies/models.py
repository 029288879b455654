"""Policies of the model zoo (one small class per model class).

Pipeline unit names per model follow Appendix-style lists of the reference policies, e.g.
cornstarch/shardformer/policies/llama.py:38-49 (``embed_tokens, rotary_emb, layers.i, norm`` and the
``model.`` prefix + ``lm_head`` for the causal-LM class), policies/siglip.py:34-46, policies/clip.py:33-44,
policies/vit.py:31-39, policies/whisper.py:36-47, policies/multimodal.py:33-44.
"""

from __future__ import annotations

from ...models import llama as L
from ...models import llama4 as L4
from ...models import phi4_audio as PA
from ...models import task_heads as H
from ...models import text_legacy as T
from ...models import vision_extra as X
from ...models import moe as M
from ...models import vision as V
from ...models import whisper as W
from ...multimodal.modeling import MultimodalProjector
from .base_policy import ModelPolicy, TPRule

_DEC_LAYER = r"(model\.)?layers\.\d+\."


class DecoderModelPolicy(ModelPolicy):
    model_cls = L.DecoderModel
    first_stage_modules = ["embed_tokens", "rotary_emb", "rotary_emb_local"]
    last_stage_modules = ["norm"]
    supported_sp_modes = ("all_to_all", "ring_attn")
    head_modules = _DEC_LAYER + r"self_attn"
    tp_rules = [
        TPRule(_DEC_LAYER + r"self_attn\.(q_proj|k_proj|v_proj)", "col"),
        TPRule(_DEC_LAYER + r"self_attn\.qkv_proj", "col", "qkv"),
        TPRule(_DEC_LAYER + r"self_attn\.o_proj", "row"),
        TPRule(_DEC_LAYER + r"mlp\.(gate_proj|up_proj)", "col"),
        TPRule(_DEC_LAYER + r"mlp\.gate_up_proj", "col", "gate_up"),
        TPRule(_DEC_LAYER + r"mlp\.down_proj", "row"),
        TPRule(_DEC_LAYER + r"(block_sparse_moe|mlp)\.experts\.\d+\.(w1|w3|gate_proj|up_proj)", "col"),
        TPRule(_DEC_LAYER + r"(block_sparse_moe|mlp)\.experts\.\d+\.(w2|down_proj)", "row"),
        TPRule(r"(model\.)?embed_tokens", "vocab"),
        TPRule(r"lm_head", "lm_head"),
    ]

    def split_sizes(self, path, module):
        cfg = self.model.config
        if path.endswith("qkv_proj"):
            d = cfg.head_dim
            return [cfg.num_attention_heads * d, cfg.num_key_value_heads * d, cfg.num_key_value_heads * d]
        if path.endswith("gate_up_proj"):
            return [cfg.intermediate_size, cfg.intermediate_size]
        return None

    def config_sanity_check(self):
        super().config_sanity_check()
        sc, cfg = self.shard_config, self.model.config
        if sc is None:
            return
        tp = sc.tensor_parallel_size
        assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0, (
            "The number of attention heads and key/value heads must be divisible by the tensor parallel size.")
        if sc.sequence_parallelism_mode == "all_to_all":
            sp = sc.sequence_parallel_size
            assert (cfg.num_attention_heads // tp) % sp == 0 and (cfg.num_key_value_heads // tp) % sp == 0, (
                "Ulysses needs the per-tp-rank head counts to be divisible by the sequence parallel size.")


class DecoderForCausalLMPolicy(DecoderModelPolicy):
    model_cls = L.DecoderForCausalLM
    first_stage_modules = ["model.embed_tokens", "model.rotary_emb", "model.rotary_emb_local"]
    last_stage_modules = ["model.norm", "lm_head"]

    def get_shared_params(self):
        cfg = self.model.config
        if getattr(cfg, "tie_word_embeddings", False):
            return [{"first": "model.embed_tokens.weight", "last": "lm_head.weight"}]
        return []


class MoeForCausalLMPolicy(DecoderForCausalLMPolicy):
    """Mixtral and Qwen3-MoE.  Both run under Ulysses and ring attention (the reference refuses sequence parallelism
    for Qwen3-MoE, cornstarch/shardformer/policies/qwen3_moe.py:107-111; here the expert block works on whatever token
    subset a rank holds, so nothing stands in the way)."""

    model_cls = M.MoeForCausalLM


_ENC_ATTN_COL = r"(q_proj|k_proj|v_proj|query|key|value)"


class SiglipVisionModelPolicy(ModelPolicy):
    model_cls = V.SiglipVisionModel
    first_stage_modules = ["vision_model.embeddings"]
    last_stage_modules = ["vision_model.post_layernorm", "vision_model.head"]
    supported_sp_modes = ("ring_attn",)
    head_modules = r"vision_model\.encoder\.layers\.\d+\.self_attn"
    tp_rules = [
        TPRule(r"vision_model\.encoder\.layers\.\d+\.self_attn\." + _ENC_ATTN_COL, "col"),
        TPRule(r"vision_model\.encoder\.layers\.\d+\.self_attn\.out_proj", "row"),
        TPRule(r"vision_model\.encoder\.layers\.\d+\.mlp\.fc1", "col"),
        TPRule(r"vision_model\.encoder\.layers\.\d+\.mlp\.fc2", "row"),
        TPRule(r"vision_model\.head\.mlp\.fc1", "col"),
        TPRule(r"vision_model\.head\.mlp\.fc2", "row"),
    ]


class CLIPVisionModelPolicy(SiglipVisionModelPolicy):
    model_cls = V.CLIPVisionModel
    first_stage_modules = ["vision_model.embeddings", "vision_model.pre_layrnorm"]
    last_stage_modules = ["vision_model.post_layernorm"]


class ViTModelPolicy(ModelPolicy):
    model_cls = V.ViTModel
    first_stage_modules = ["embeddings"]
    last_stage_modules = ["layernorm", "pooler"]
    supported_sp_modes = ("ring_attn",)
    head_modules = r"encoder\.layer\.\d+"
    tp_rules = [
        TPRule(r"encoder\.layer\.\d+\.attention\.attention\." + _ENC_ATTN_COL, "col"),
        TPRule(r"encoder\.layer\.\d+\.attention\.output\.dense", "row"),
        TPRule(r"encoder\.layer\.\d+\.intermediate\.dense", "col"),
        TPRule(r"encoder\.layer\.\d+\.output\.dense", "row"),
    ]


class WhisperEncoderPolicy(ModelPolicy):
    model_cls = W.WhisperEncoder
    first_stage_modules = ["conv1", "conv2", "embed_positions"]
    last_stage_modules = ["layer_norm", "avg_pooler"]
    supported_sp_modes = ("ring_attn",)
    head_modules = r"layers\.\d+\.self_attn"
    tp_rules = [
        TPRule(r"layers\.\d+\.self_attn\." + _ENC_ATTN_COL, "col"),
        TPRule(r"layers\.\d+\.self_attn\.out_proj", "row"),
        TPRule(r"layers\.\d+\.fc1", "col"),
        TPRule(r"layers\.\d+\.fc2", "row"),
    ]


class Qwen2AudioEncoderPolicy(WhisperEncoderPolicy):
    model_cls = W.Qwen2AudioEncoder


class MultimodalProjectorPolicy(ModelPolicy):
    """``linear`` -> column-parallel with gathered output; ``in_proj`` column, ``out_proj`` row."""

    model_cls = MultimodalProjector
    tp_rules = [
        TPRule(r"projection\.linear", "col_gather"),
        TPRule(r"projection\.in_proj", "col"),
        TPRule(r"projection\.out_proj", "row"),
    ]

    @classmethod
    def get_all_modules(cls, config) -> list[str]:
        return MultimodalProjector.module_names(config)

    def pipeline_template_sanity_check(self, template) -> None:
        return None


class Dinov2ModelPolicy(ViTModelPolicy):
    model_cls = X.Dinov2Model
    last_stage_modules = ["layernorm"]
    tp_rules = [
        TPRule(r"encoder\.layer\.\d+\.attention\.attention\." + _ENC_ATTN_COL, "col"),
        TPRule(r"encoder\.layer\.\d+\.attention\.output\.dense", "row"),
        TPRule(r"encoder\.layer\.\d+\.mlp\.fc1", "col"),
        TPRule(r"encoder\.layer\.\d+\.mlp\.fc2", "row"),
    ]


class EvaCLIPVisionModelPolicy(SiglipVisionModelPolicy):
    model_cls = X.EvaCLIPVisionModel
    last_stage_modules = ["vision_model.post_layernorm"]
    head_modules = r"vision_model\.encoder\.layers\.\d+"
    tp_rules = SiglipVisionModelPolicy.tp_rules[:4]


class InternVisionModelPolicy(ModelPolicy):
    """Pipeline only when q/k are RMS-normalised over the full width (that norm cannot be sharded); otherwise the
    fused qkv is column parallel (cornstarch/shardformer/policies/intern_vit.py:35-45)."""

    model_cls = X.InternVisionModel
    supported_sp_modes = ("ring_attn",)  # the reference switches sequence parallelism off for this model (intern_vit.py:82-83)
    first_stage_modules = ["embeddings"]
    last_stage_modules = []
    head_modules = r"encoder\.layers\.\d+"
    tp_rules = [
        TPRule(r"encoder\.layers\.\d+\.attn\.qkv", "col", "qkv"),
        TPRule(r"encoder\.layers\.\d+\.attn\.proj", "row"),
        TPRule(r"encoder\.layers\.\d+\.mlp\.fc1", "col"),
        TPRule(r"encoder\.layers\.\d+\.mlp\.fc2", "row"),
    ]

    def split_sizes(self, path, module):
        H = self.model.config.hidden_size
        return [H, H, H] if path.endswith("qkv") else None

    def config_sanity_check(self):
        super().config_sanity_check()
        sc = self.shard_config
        if sc is not None and sc.tensor_parallel_size > 1 and self.model.config.qk_normalization:
            raise ValueError("InternViT with qk_normalization cannot be tensor parallel: q_norm/k_norm span all heads")


class PixtralVisionModelPolicy(ModelPolicy):
    model_cls = X.PixtralVisionModel
    first_stage_modules = ["patch_conv", "ln_pre", "patch_positional_embedding"]
    last_stage_modules = []
    supported_sp_modes = ("ring_attn",)
    head_modules = r"transformer\.layers\.\d+"
    tp_rules = [
        TPRule(r"transformer\.layers\.\d+\.attention\.(q_proj|k_proj|v_proj)", "col"),
        TPRule(r"transformer\.layers\.\d+\.attention\.o_proj", "row"),
        TPRule(r"transformer\.layers\.\d+\.feed_forward\.(gate_proj|up_proj)", "col"),
        TPRule(r"transformer\.layers\.\d+\.feed_forward\.down_proj", "row"),
    ]


class Qwen2VisionTransformerPolicy(ModelPolicy):
    model_cls = X.Qwen2VisionTransformerPretrainedModel
    first_stage_modules = ["patch_embed", "rotary_pos_emb"]
    last_stage_modules = ["merger"]
    supported_sp_modes = ("ring_attn",)  # tokens are split per image in whole 2 x 2 merge groups
    head_modules = r"blocks\.\d+"
    tp_rules = [
        TPRule(r"blocks\.\d+\.attn\.qkv", "col", "qkv"),
        TPRule(r"blocks\.\d+\.attn\.proj", "row"),
        TPRule(r"blocks\.\d+\.mlp\.fc1", "col"),
        TPRule(r"blocks\.\d+\.mlp\.fc2", "row"),
    ]

    def split_sizes(self, path, module):
        H = self.model.config.embed_dim
        return [H, H, H] if path.endswith("qkv") else None


class GPT2ModelPolicy(ModelPolicy):
    """GPT-2 stores its projection weights transposed (``Conv1D``): ``c_attn`` (fused q, k, v) and ``c_fc`` are split
    over their output features, the two ``c_proj`` over their input features (module list
    cornstarch/shardformer/policies/gpt2.py:44-55).  Embeddings and the LM head stay replicated."""

    model_cls = T.GPT2Model
    first_stage_modules = ["wte", "wpe", "drop"]
    last_stage_modules = ["ln_f"]
    head_modules = r"(transformer\.)?h\.\d+"
    tp_rules = [
        TPRule(r"(transformer\.)?h\.\d+\.attn\.c_attn", "col", "qkv"),
        TPRule(r"(transformer\.)?h\.\d+\.attn\.c_proj", "row"),
        TPRule(r"(transformer\.)?h\.\d+\.mlp\.c_fc", "col"),
        TPRule(r"(transformer\.)?h\.\d+\.mlp\.c_proj", "row"),
    ]

    def split_sizes(self, path, module):
        H = self.model.config.n_embd
        return [H, H, H] if path.endswith("c_attn") else None


class GPT2LMHeadModelPolicy(GPT2ModelPolicy):
    model_cls = T.GPT2LMHeadModel
    first_stage_modules = ["transformer.wte", "transformer.wpe", "transformer.drop"]
    last_stage_modules = ["transformer.ln_f", "lm_head"]

    def get_shared_params(self):
        if getattr(self.model.config, "tie_word_embeddings", False):
            return [{"first": "transformer.wte.weight", "last": "lm_head.weight"}]
        return []


class BertModelPolicy(ModelPolicy):
    model_cls = T.BertModel
    first_stage_modules = ["embeddings"]
    last_stage_modules = ["pooler"]
    head_modules = r"(bert\.)?encoder\.layer\.\d+"
    tp_rules = [
        TPRule(r"(bert\.)?encoder\.layer\.\d+\.attention\.self\.(query|key|value)", "col"),
        TPRule(r"(bert\.)?encoder\.layer\.\d+\.attention\.output\.dense", "row"),
        TPRule(r"(bert\.)?encoder\.layer\.\d+\.intermediate\.dense", "col"),
        TPRule(r"(bert\.)?encoder\.layer\.\d+\.output\.dense", "row"),
    ]


class BertForMaskedLMPolicy(BertModelPolicy):
    model_cls = T.BertForMaskedLM
    first_stage_modules = ["bert.embeddings"]
    last_stage_modules = ["cls"]


class OPTModelPolicy(ModelPolicy):
    model_cls = T.OPTModel
    first_stage_modules = ["decoder.embed_tokens", "decoder.embed_positions", "decoder.project_in"]
    last_stage_modules = ["decoder.final_layer_norm", "decoder.project_out"]
    head_modules = r"(model\.)?decoder\.layers\.\d+"
    tp_rules = [
        TPRule(r"(model\.)?decoder\.layers\.\d+\.self_attn\.(q_proj|k_proj|v_proj)", "col"),
        TPRule(r"(model\.)?decoder\.layers\.\d+\.self_attn\.out_proj", "row"),
        TPRule(r"(model\.)?decoder\.layers\.\d+\.fc1", "col"),
        TPRule(r"(model\.)?decoder\.layers\.\d+\.fc2", "row"),
    ]


class OPTForCausalLMPolicy(OPTModelPolicy):
    model_cls = T.OPTForCausalLM
    first_stage_modules = ["model.decoder.embed_tokens", "model.decoder.embed_positions", "model.decoder.project_in"]
    last_stage_modules = ["model.decoder.final_layer_norm", "model.decoder.project_out", "lm_head"]


_L4_LAYER = r"(model\.)?layers\.\d+\."


class Llama4TextModelPolicy(ModelPolicy):
    """Attention and the shared expert / dense MLP are tensor parallel; the stacked routed experts stay replicated
    (cornstarch/shardformer/policies/llama4.py:188-218 shards attention + shared_expert the same way)."""

    model_cls = L4.Llama4TextModel
    first_stage_modules = ["embed_tokens", "rotary_emb"]
    last_stage_modules = ["norm"]
    supported_sp_modes = ("all_to_all", "ring_attn")  # both with the plain causal mask
    head_modules = _L4_LAYER + r"self_attn"
    tp_rules = [
        TPRule(_L4_LAYER + r"self_attn\.(q_proj|k_proj|v_proj)", "col"),
        TPRule(_L4_LAYER + r"self_attn\.o_proj", "row"),
        TPRule(_L4_LAYER + r"feed_forward\.(shared_expert\.)?(gate_proj|up_proj)", "col"),
        TPRule(_L4_LAYER + r"feed_forward\.(shared_expert\.)?down_proj", "row"),
        TPRule(r"(model\.)?embed_tokens", "vocab"),
        TPRule(r"lm_head", "lm_head"),
    ]


class Llama4ForCausalLMPolicy(Llama4TextModelPolicy):
    model_cls = L4.Llama4ForCausalLM
    first_stage_modules = ["model.embed_tokens", "model.rotary_emb"]
    last_stage_modules = ["model.norm", "lm_head"]


class Phi4MultimodalAudioModelPolicy(ModelPolicy):
    model_cls = PA.Phi4MultimodalAudioModel
    first_stage_modules = ["encoder_embedding", "embed", "relative_attention_bias_layer"]
    last_stage_modules = []
    head_modules = r"encoders\.\d+\.self_attn"
    supported_sp_modes = ("ring_attn", "all_to_all")  # contiguous chunks; the causal convolutions exchange a halo
    tp_rules = [
        TPRule(r"encoders\.\d+\.self_attn\.(q_proj|k_proj|v_proj)", "col"),
        TPRule(r"encoders\.\d+\.self_attn\.o_proj", "row"),
        TPRule(r"encoders\.\d+\.feed_forward_(in|out)\.gate_up_proj", "col"),
        TPRule(r"encoders\.\d+\.feed_forward_(in|out)\.down_proj", "row"),
    ]

    def split_sizes(self, path, module):
        I = self.model.config.intermediate_size
        return [I, I] if path.endswith("gate_up_proj") else None


# ------------------------------------------------------------------------------------------------ task heads
# Pipeline units of the head classes: the backbone's units under its prefix plus the head units, which must sit on the
# last stage (cornstarch/shardformer/policies/bert.py:106-260, gpt2.py:97-180, opt.py:99-135, dinov2.py:254-259).
class BertForPreTrainingPolicy(BertModelPolicy):
    model_cls = H.BertForPreTraining
    first_stage_modules = ["bert.embeddings"]
    last_stage_modules = ["cls"]


class BertLMHeadModelPolicy(BertForPreTrainingPolicy):
    model_cls = H.BertLMHeadModel


class BertForNextSentencePredictionPolicy(BertForPreTrainingPolicy):
    model_cls = H.BertForNextSentencePrediction


class BertForSequenceClassificationPolicy(BertModelPolicy):
    model_cls = H.BertForSequenceClassification
    first_stage_modules = ["bert.embeddings"]
    last_stage_modules = ["dropout", "classifier"]


class BertForTokenClassificationPolicy(BertForSequenceClassificationPolicy):
    model_cls = H.BertForTokenClassification


class BertForMultipleChoicePolicy(BertForSequenceClassificationPolicy):
    model_cls = H.BertForMultipleChoice


class BertForQuestionAnsweringPolicy(BertModelPolicy):
    model_cls = H.BertForQuestionAnswering
    first_stage_modules = ["bert.embeddings"]
    last_stage_modules = ["qa_outputs"]


class GPT2DoubleHeadsModelPolicy(GPT2LMHeadModelPolicy):
    model_cls = H.GPT2DoubleHeadsModel
    last_stage_modules = ["transformer.ln_f", "lm_head", "multiple_choice_head"]


class GPT2ForQuestionAnsweringPolicy(GPT2ModelPolicy):
    model_cls = H.GPT2ForQuestionAnswering
    first_stage_modules = ["transformer.wte", "transformer.wpe", "transformer.drop"]
    last_stage_modules = ["transformer.ln_f", "qa_outputs"]


class GPT2ForTokenClassificationPolicy(GPT2ForQuestionAnsweringPolicy):
    model_cls = H.GPT2ForTokenClassification
    last_stage_modules = ["transformer.ln_f", "dropout", "classifier"]


class GPT2ForSequenceClassificationPolicy(GPT2ForQuestionAnsweringPolicy):
    model_cls = H.GPT2ForSequenceClassification
    last_stage_modules = ["transformer.ln_f", "score"]


class OPTForSequenceClassificationPolicy(OPTForCausalLMPolicy):
    model_cls = H.OPTForSequenceClassification
    last_stage_modules = ["model.decoder.final_layer_norm", "model.decoder.project_out", "score"]


class OPTForQuestionAnsweringPolicy(OPTForCausalLMPolicy):
    model_cls = H.OPTForQuestionAnswering
    last_stage_modules = ["model.decoder.final_layer_norm", "model.decoder.project_out", "qa_outputs"]


class DecoderForSequenceClassificationPolicy(DecoderModelPolicy):
    """``LlamaForSequenceClassification``: the decoder's units under ``model.`` plus ``score`` on the last stage."""

    model_cls = H.DecoderForSequenceClassification
    first_stage_modules = ["model.embed_tokens", "model.rotary_emb", "model.rotary_emb_local"]
    last_stage_modules = ["model.norm", "score"]


class Dinov2BackbonePolicy(Dinov2ModelPolicy):
    model_cls = H.Dinov2Backbone


class Dinov2ForImageClassificationPolicy(Dinov2ModelPolicy):
    model_cls = H.Dinov2ForImageClassification
    first_stage_modules = ["dinov2.embeddings"]
    last_stage_modules = ["dinov2.layernorm", "classifier"]
    head_modules = r"dinov2\.encoder\.layer\.\d+"
    tp_rules = [TPRule(r"dinov2\." + r.pattern, r.kind, r.split_sizes_attr) for r in Dinov2ModelPolicy.tp_rules]


# The per-family names the reference uses (``LlamaForCausalLMPolicy``, ``MixtralModelPolicy``, ...;
# cornstarch/shardformer/policies/<family>.py).  The decoder families share one implementation here: the differences
# between them are in the model's spec, not in how it is sharded.
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
