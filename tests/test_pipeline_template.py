"""PipelineTemplate: module lists per model class, layer counting, sanity checks, hashing
(reference: tests/test_pipeline_template.py:23-117)."""

import pytest
import torch

from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM, DecoderModel
from cornstarch_b200.models.vision import CLIPVisionConfig, CLIPVisionModel, SiglipVisionConfig, SiglipVisionModel, ViTConfig, ViTModel
from cornstarch_b200.models.whisper import WhisperConfig, WhisperEncoder
from cornstarch_b200.multimodal.modeling import ModalEncoderModule, MultimodalProjector, MultimodalProjectorConfig
from cornstarch_b200.pipeline_template import PipelineTemplate
from cornstarch_b200.shardformer.policies.auto_policy import get_autopolicy, policy_for_model

CFG = DecoderConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4)


def test_module_names_per_family():
    with torch.device("meta"):
        llm = DecoderForCausalLM(CFG)
        base = DecoderModel(CFG)
        sig = SiglipVisionModel(SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14))
        clip = CLIPVisionModel(CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14))
        vit = ViTModel(ViTConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14))
        wh = WhisperEncoder(WhisperConfig(num_mel_bins=8, d_model=32, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=64, max_source_positions=10))
    assert PipelineTemplate.get_modules(base) == ["embed_tokens", "rotary_emb", "layers.0", "layers.1", "layers.2", "layers.3", "norm"]
    assert PipelineTemplate.get_modules(llm) == ["model.embed_tokens", "model.rotary_emb", "model.layers.0", "model.layers.1",
                                                 "model.layers.2", "model.layers.3", "model.norm", "lm_head"]
    assert PipelineTemplate.get_modules(sig) == ["vision_model.embeddings", "vision_model.encoder.layers.0", "vision_model.encoder.layers.1",
                                                 "vision_model.post_layernorm", "vision_model.head"]
    assert PipelineTemplate.get_modules(clip) == ["vision_model.embeddings", "vision_model.pre_layrnorm", "vision_model.encoder.layers.0",
                                                  "vision_model.encoder.layers.1", "vision_model.post_layernorm"]
    assert PipelineTemplate.get_modules(vit) == ["embeddings", "encoder.layer.0", "encoder.layer.1", "layernorm", "pooler"]
    assert PipelineTemplate.get_modules(wh) == ["conv1", "conv2", "embed_positions", "layers.0", "layers.1", "layer_norm"]


def test_modal_module_names_and_even_split():
    with torch.device("meta"):
        vit = ViTModel(ViTConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4, image_size=28, patch_size=14))
        llm = DecoderForCausalLM(CFG)
        proj = MultimodalProjector(MultimodalProjectorConfig(encoder_config=vit.config, text_config=CFG, projection_type="mlp"))
        lin = MultimodalProjector(MultimodalProjectorConfig(encoder_config=vit.config, text_config=CFG, projection_type="linear"))
    enc = ModalEncoderModule(vit, proj)
    names = PipelineTemplate.get_modules(enc)
    assert names[0] == "module.embeddings" and names[-3:] == ["projector.in_proj", "projector.activation", "projector.out_proj"]
    assert PipelineTemplate.get_modules(ModalEncoderModule(vit, lin))[-1] == "projector.projection"
    t = PipelineTemplate.even_split(enc, 2)
    assert t.num_stages == 2 and t.get_num_layers_per_stage() == [2, 2]
    assert t.modules_per_stage[0][0] == "module.embeddings" and t.modules_per_stage[1][-1] == "projector.out_proj"
    t3 = PipelineTemplate.even_split(llm, 3)
    assert t3.get_num_layers_per_stage() == [2, 1, 1] and t3.modules_per_stage[-1][-1] == "lm_head"
    assert t3.num_layers == 8


def test_latency_hash_eq_find():
    a = PipelineTemplate("m", [["layers.0"], ["layers.1"]], latency=10.0, kstar_latency=2.0)
    b = PipelineTemplate("m", [["layers.0"], ["layers.1"]])
    c = PipelineTemplate("m", [["layers.0", "layers.1"]])
    assert a == b and hash(a) == hash(b) and a != c
    assert a.latency(10) == 10.0 + 2.0 * (10 - 8)
    with pytest.raises(AssertionError):
        a.latency(1)
    assert PipelineTemplate.find_pipeline_template([a, c], 1) is c and PipelineTemplate.find_pipeline_template([a, c], 3) is None


def test_sanity_check_rejects_bad_templates():
    with torch.device("meta"):
        llm = DecoderForCausalLM(CFG)
    pol = policy_for_model(llm)
    names = PipelineTemplate.get_modules(llm)
    pol.pipeline_template_sanity_check(PipelineTemplate("x", [names[:4], names[4:]]))
    with pytest.raises(ValueError):  # a module is missing
        pol.pipeline_template_sanity_check(PipelineTemplate("x", [names[:4], names[5:]]))
    with pytest.raises(ValueError):  # lm_head not on the last stage
        pol.pipeline_template_sanity_check(PipelineTemplate("x", [names[:4] + ["lm_head"], names[4:-1]]))


def test_autopolicy_resolves_hf_names():
    p = get_autopolicy("transformers.models.llama.modeling_llama.LlamaForCausalLM")
    assert type(p).get_all_modules(CFG)[-1] == "lm_head"
    with pytest.raises(NotImplementedError):
        get_autopolicy("nowhere.Model")
