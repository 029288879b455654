"""Composite HF checkpoints -> MultimodalModel: the state dict of a (tiny, random) LLaVA-NeXT / Qwen2-VL model is cut into
vision tower, projector and language model; the parts reproduce the HF sub-modules' outputs."""

import pytest
import torch

tf = pytest.importorskip("transformers")


def test_llava_next_split_and_forward():
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaNextConfig, LlavaNextForConditionalGeneration

    from cornstarch_b200.multimodal.adapters import multimodal_from_state_dict

    torch.manual_seed(0)
    cfg = LlavaNextConfig(
        vision_config=CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28,
                                       patch_size=14).to_dict(),
        text_config=LlamaConfig(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2).to_dict(),
        image_token_index=199, image_grid_pinpoints=[[28, 28]])
    hf = LlavaNextForConditionalGeneration(cfg).eval()
    model = multimodal_from_state_dict("llava_next", cfg.to_dict(), hf.state_dict()).eval()
    assert model.token_ids == {"vision": 199}
    px = torch.randn(2, 3, 28, 28)
    # vision tower at feature layer -2 without the CLS token, then the 2-layer projector
    with torch.no_grad():
        hs = hf.model.vision_tower(px, output_hidden_states=True).hidden_states[-2][:, 1:]
        want = hf.model.multi_modal_projector(hs)
        got = model.vision_encoder(pixel_values=px)
    got = got["hidden_states"] if isinstance(got, dict) else got[0]
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()
    # language model alone
    ids = torch.randint(0, 198, (2, 12))
    with torch.no_grad():
        a = hf.lm_head(hf.model.language_model(input_ids=ids).last_hidden_state)
        b = model.language_model(input_ids=ids).logits
    assert torch.allclose(a, b, atol=1e-4)
    # full multimodal forward: 4 image placeholders per sample
    ids2 = torch.cat([torch.full((2, 4), 199), ids], dim=1)
    out = model(input_ids=ids2, pixel_values=px, labels=ids2)
    assert torch.isfinite(out.loss)


def test_qwen2_vl_split():
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    from cornstarch_b200.multimodal.adapters import multimodal_from_state_dict

    torch.manual_seed(0)
    vc = dict(depth=2, embed_dim=32, hidden_size=48, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    tc = dict(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              rope_scaling={"type": "mrope", "mrope_section": [2, 2, 2]})
    try:
        cfg = Qwen2VLConfig(vision_config=vc, text_config=tc, image_token_id=199)
    except TypeError:
        cfg = Qwen2VLConfig(vision_config=vc, image_token_id=199, **tc)
    hf = Qwen2VLForConditionalGeneration(cfg).eval()
    d = cfg.to_dict()
    model = multimodal_from_state_dict("qwen2_vl", d, hf.state_dict()).eval()
    grid = torch.tensor([[1, 4, 4]])
    x = torch.randn(16, 3 * 2 * 14 * 14)
    with torch.no_grad():
        visual = hf.model.visual if hasattr(hf.model, "visual") else hf.visual
        want = visual(x, grid_thw=grid)
        want = want if isinstance(want, torch.Tensor) else (want.pooler_output if getattr(want, "pooler_output", None) is not None else want[0])
        got = model.vision_encoder(hidden_states=x, grid_thw=grid)
    got = got["hidden_states"] if isinstance(got, dict) else got[0]
    assert torch.allclose(got.reshape(want.shape), want, atol=1e-4), (got.reshape(want.shape) - want).abs().max()


def test_llava_next_from_a_checkpoint_directory(tmp_path):
    """``MultimodalModel.from_pretrained_multimodal_model(dir)`` on a directory written by ``transformers``."""
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaNextConfig, LlavaNextForConditionalGeneration

    from cornstarch_b200.multimodal import MultimodalModel

    torch.manual_seed(0)
    cfg = LlavaNextConfig(
        vision_config=CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28,
                                       patch_size=14).to_dict(),
        text_config=LlamaConfig(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2).to_dict(),
        image_token_index=199, image_grid_pinpoints=[[28, 28]])
    hf = LlavaNextForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path))
    model = MultimodalModel.from_pretrained_multimodal_model(str(tmp_path)).eval()
    assert model.token_ids == {"vision": 199}
    ids = torch.randint(0, 198, (2, 12))
    with torch.no_grad():
        a = hf.lm_head(hf.model.language_model(input_ids=ids).last_hidden_state)
        b = model.language_model(input_ids=ids).logits
    assert torch.allclose(a, b, atol=1e-4)


def test_qwen2_vl_from_a_checkpoint_directory(tmp_path):
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration

    from cornstarch_b200.multimodal import MultimodalModel

    torch.manual_seed(0)
    vc = dict(depth=2, embed_dim=32, hidden_size=48, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    tc = dict(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              rope_scaling={"type": "mrope", "mrope_section": [2, 2, 2]})
    try:
        cfg = Qwen2VLConfig(vision_config=vc, text_config=tc, image_token_id=199)
    except TypeError:
        cfg = Qwen2VLConfig(vision_config=vc, image_token_id=199, **tc)
    hf = Qwen2VLForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path))
    model = MultimodalModel.from_pretrained_multimodal_model(str(tmp_path)).eval()
    assert model.token_ids == {"vision": 199}
    grid = torch.tensor([[1, 4, 4]])
    x = torch.randn(16, 3 * 2 * 14 * 14)
    with torch.no_grad():
        visual = hf.model.visual if hasattr(hf.model, "visual") else hf.visual
        want = visual(x, grid_thw=grid)
        want = want if isinstance(want, torch.Tensor) else (want.pooler_output if getattr(want, "pooler_output", None) is not None else want[0])
        got = model.vision_encoder(hidden_states=x, grid_thw=grid)
    got = got["hidden_states"] if isinstance(got, dict) else got[0]
    assert torch.allclose(got.reshape(want.shape), want, atol=1e-4)


def test_language_model_alone_from_a_llava_checkpoint(tmp_path):
    """The decoder of a vision-language checkpoint loads on its own: nested ``text_config``, the ``model.language_model.``
    prefix, and the head that the same file keeps under ``language_model.lm_head``."""
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaNextConfig, LlavaNextForConditionalGeneration

    from cornstarch_b200.models.llama import DecoderForCausalLM

    torch.manual_seed(0)
    cfg = LlavaNextConfig(
        vision_config=CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=28,
                                       patch_size=14).to_dict(),
        text_config=LlamaConfig(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2).to_dict(),
        image_token_index=199, image_grid_pinpoints=[[28, 28]])
    hf = LlavaNextForConditionalGeneration(cfg).eval()
    hf.save_pretrained(str(tmp_path))
    llm = DecoderForCausalLM.from_pretrained(str(tmp_path)).eval()
    ids = torch.randint(0, 198, (2, 12))
    with torch.no_grad():
        want = hf.lm_head(hf.model.language_model(input_ids=ids).last_hidden_state)
        assert torch.allclose(llm(input_ids=ids).logits, want, atol=1e-4)


@pytest.mark.parametrize("tower", ["clip", "siglip"])
def test_llava_full_forward_matches_hf(tower):
    """LLaVA-1.5 (CLIP tower, CLS dropped) and its SigLIP variant (all patch tokens): logits of the whole multimodal
    forward equal those of ``LlavaForConditionalGeneration`` with the same weights."""
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaConfig, LlavaForConditionalGeneration, SiglipVisionConfig

    from cornstarch_b200.multimodal.adapters import multimodal_from_state_dict

    torch.manual_seed(0)
    vkw = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=14)
    vision = CLIPVisionConfig(**vkw) if tower == "clip" else SiglipVisionConfig(**vkw)
    cfg = LlavaConfig(
        vision_config=vision.to_dict(),
        text_config=LlamaConfig(vocab_size=200, hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2).to_dict(),
        image_token_index=199, vision_feature_layer=-2, vision_feature_select_strategy="default" if tower == "clip" else "full")
    hf = LlavaForConditionalGeneration(cfg).eval()
    model = multimodal_from_state_dict("llava", cfg.to_dict(), hf.state_dict()).eval()
    model.mask_mode = "causal"  # image tokens attend causally in Hugging Face's LLaVA
    px = torch.randn(2, 3, 28, 28)
    ids = torch.cat([torch.randint(0, 198, (2, 3)), torch.full((2, 4), 199), torch.randint(0, 198, (2, 9))], dim=1)
    with torch.no_grad():
        want = hf(input_ids=ids, pixel_values=px).logits
        got = model(input_ids=ids, pixel_values=px).logits
    assert torch.allclose(got, want, atol=2e-4), (got - want).abs().max()
