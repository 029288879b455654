"""Checkpoint format: a directory written by ``save_pretrained`` here loads in Hugging Face ``transformers`` and gives the
same outputs, and a directory written by ``transformers`` loads here."""

import pytest
import torch

tf = pytest.importorskip("transformers")

KW = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
          num_key_value_heads=2, max_position_embeddings=64)


def _decoder(family):
    from cornstarch_b200.models import llama as L
    from cornstarch_b200.models import moe as M

    if family == "mixtral":
        return M.MoeForCausalLM(M.MixtralConfig(**KW, num_local_experts=4, num_experts_per_tok=2)), tf.MixtralForCausalLM
    cfg_cls, hf_cls, extra = {
        "llama": (L.LlamaConfig, tf.LlamaForCausalLM, {}),
        "mistral": (L.MistralConfig, tf.MistralForCausalLM, {}),
        "qwen2": (L.Qwen2Config, tf.Qwen2ForCausalLM, {}),
        "qwen3": (L.Qwen3Config, tf.Qwen3ForCausalLM, dict(head_dim=16)),
        "phi3": (L.Phi3Config, tf.Phi3ForCausalLM, dict(pad_token_id=0)),
    }[family]
    return L.DecoderForCausalLM(cfg_cls(**KW, **extra)), hf_cls


@pytest.mark.parametrize("family", ["llama", "mistral", "qwen2", "qwen3", "phi3", "mixtral"])
def test_decoder_checkpoints_round_trip_through_transformers(family, tmp_path):
    torch.manual_seed(0)
    mine, hf_cls = _decoder(family)
    mine.eval()
    mine.save_pretrained(str(tmp_path / "ours"))
    hf = hf_cls.from_pretrained(str(tmp_path / "ours")).eval()
    ids = torch.randint(0, 128, (2, 16))
    with torch.no_grad():
        want = mine(input_ids=ids).logits
        assert torch.allclose(hf(input_ids=ids).logits, want, atol=1e-4)
    hf.save_pretrained(str(tmp_path / "theirs"))
    back = type(mine).from_pretrained(str(tmp_path / "theirs")).eval()
    with torch.no_grad():
        assert torch.allclose(back(input_ids=ids).logits, want, atol=1e-5)


def test_vision_checkpoints_round_trip_through_transformers(tmp_path):
    from cornstarch_b200.models import vision as V

    torch.manual_seed(0)
    common = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    px = torch.randn(2, 3, 28, 28)
    for name, mine, hf_cls in (("siglip", V.SiglipVisionModel(V.SiglipVisionConfig(**common)), tf.SiglipVisionModel),
                               ("clip", V.CLIPVisionModel(V.CLIPVisionConfig(**common)), tf.CLIPVisionModel),
                               ("vit", V.ViTModel(V.ViTConfig(**common)), tf.ViTModel)):
        mine.eval()
        mine.save_pretrained(str(tmp_path / name))
        hf = hf_cls.from_pretrained(str(tmp_path / name)).eval()
        with torch.no_grad():
            a, b = hf(pixel_values=px).last_hidden_state, mine(pixel_values=px).last_hidden_state
        assert torch.allclose(a, b, atol=1e-4), (name, (a - b).abs().max())


def test_auto_model_picks_the_family_from_the_checkpoint(tmp_path):
    from cornstarch_b200.models import AutoModel

    torch.manual_seed(0)
    hf = tf.Qwen3ForCausalLM(tf.Qwen3Config(**KW, head_dim=16)).eval()
    hf.save_pretrained(str(tmp_path))
    mine = AutoModel.from_pretrained(str(tmp_path)).eval()
    assert hasattr(mine.model.layers[0].self_attn, "q_norm")
    ids = torch.randint(0, 128, (1, 12))
    with torch.no_grad():
        assert torch.allclose(mine(input_ids=ids).logits, hf(input_ids=ids).logits, atol=1e-4)


@pytest.mark.parametrize("family", ["gemma", "gemma2", "qwen3_moe", "gpt2", "opt", "dinov2"])
def test_auto_model_loads_transformers_checkpoints(family, tmp_path):
    """A directory written by ``transformers`` loads through ``AutoModel`` without missing or unexpected tensors and gives
    the same output."""
    from cornstarch_b200.models import AutoModel

    torch.manual_seed(0)
    ids = torch.randint(0, 128, (2, 12))
    if family == "gemma":
        hf = tf.GemmaForCausalLM(tf.GemmaConfig(**KW, head_dim=16, hidden_activation="gelu_pytorch_tanh"))
    elif family == "gemma2":
        hf = tf.Gemma2ForCausalLM(tf.Gemma2Config(**KW, head_dim=16, query_pre_attn_scalar=16, attn_logit_softcapping=None,
                                                  final_logit_softcapping=None, sliding_window=4096))
    elif family == "qwen3_moe":
        hf = tf.Qwen3MoeForCausalLM(tf.Qwen3MoeConfig(**KW, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
                                                      decoder_sparse_step=1, mlp_only_layers=[]))
    elif family == "gpt2":
        hf = tf.GPT2LMHeadModel(tf.GPT2Config(n_layer=2, n_embd=64, n_head=4, vocab_size=128, n_positions=64))
    elif family == "opt":
        hf = tf.OPTForCausalLM(tf.OPTConfig(vocab_size=128, hidden_size=64, ffn_dim=128, num_hidden_layers=2, num_attention_heads=4,
                                            max_position_embeddings=64, word_embed_proj_dim=64))
    else:
        hf = tf.Dinov2Model(tf.Dinov2Config(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14))
    hf.eval()
    hf.save_pretrained(str(tmp_path))
    mine = AutoModel.from_pretrained(str(tmp_path)).eval()
    with torch.no_grad():
        if family == "dinov2":
            px = torch.randn(2, 3, 28, 28)
            a, b = hf(pixel_values=px).last_hidden_state, mine(pixel_values=px).last_hidden_state
        else:
            a, b = hf(input_ids=ids).logits, mine(input_ids=ids).logits
    assert torch.allclose(a, b, atol=2e-4), (family, (a - b).abs().max())


def test_sub_models_load_from_composite_checkpoints(tmp_path):
    """The Whisper encoder from a full Whisper checkpoint, the SigLIP vision tower from a two-tower SigLIP checkpoint: the
    key prefix and the nested config are found, the other tensors are ignored."""
    from cornstarch_b200.models import vision as V
    from cornstarch_b200.models import whisper as W

    torch.manual_seed(0)
    kw = dict(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, max_source_positions=50)
    hf = tf.WhisperForConditionalGeneration(tf.WhisperConfig(
        **kw, decoder_layers=1, decoder_attention_heads=4, decoder_ffn_dim=64, vocab_size=100, pad_token_id=0, bos_token_id=1,
        eos_token_id=2, decoder_start_token_id=1)).eval()
    hf.save_pretrained(str(tmp_path / "whisper"))
    enc = W.WhisperEncoder.from_pretrained(str(tmp_path / "whisper")).eval()
    x = torch.randn(2, 16, 100)
    with torch.no_grad():
        assert torch.allclose(enc(input_features=x).last_hidden_state, hf.model.encoder(x).last_hidden_state, atol=1e-4)

    common = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    two = tf.SiglipModel(tf.SiglipConfig(vision_config=common, text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1,
                                                                                num_attention_heads=4, vocab_size=100))).eval()
    two.save_pretrained(str(tmp_path / "siglip"))
    tower = V.SiglipVisionModel.from_pretrained(str(tmp_path / "siglip")).eval()
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        assert torch.allclose(tower(pixel_values=px).last_hidden_state, two.vision_model(pixel_values=px).last_hidden_state, atol=1e-4)


def test_more_sub_models_from_composite_checkpoints(tmp_path):
    """CLIP's vision tower from a two-tower CLIP checkpoint; the audio tower of a Qwen2-Audio checkpoint."""
    from transformers import Qwen2AudioConfig, Qwen2AudioForConditionalGeneration

    from cornstarch_b200.models import vision as V
    from cornstarch_b200.models import whisper as W

    torch.manual_seed(0)
    common = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    clip = tf.CLIPModel(tf.CLIPConfig(vision_config=common, projection_dim=32,
                                      text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4,
                                                       vocab_size=100))).eval()
    clip.save_pretrained(str(tmp_path / "clip"))
    tower = V.CLIPVisionModel.from_pretrained(str(tmp_path / "clip")).eval()
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        assert torch.allclose(tower(pixel_values=px).last_hidden_state, clip.vision_model(pixel_values=px).last_hidden_state, atol=1e-4)

    ac = dict(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, max_source_positions=50)
    tc = dict(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
              model_type="qwen2")
    qa = Qwen2AudioForConditionalGeneration(Qwen2AudioConfig(audio_config=ac, text_config=tc)).eval()
    qa.save_pretrained(str(tmp_path / "qwen2_audio"))
    enc = W.Qwen2AudioEncoder.from_pretrained(str(tmp_path / "qwen2_audio")).eval()
    x = torch.randn(2, 16, 100)
    with torch.no_grad():
        assert torch.allclose(enc(input_features=x).last_hidden_state, qa.audio_tower(x).last_hidden_state, atol=1e-4)
