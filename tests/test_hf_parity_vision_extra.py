"""DINOv2, Pixtral and the Qwen2-VL vision tower against the HF implementations (fp32, CPU); EvaCLIP and InternViT
(not in transformers) against a direct PyTorch statement of their blocks."""

import pytest
import torch
import torch.nn.functional as F

transformers = pytest.importorskip("transformers")


def _load(ours, hf_sd):
    missing, unexpected = ours.load_state_dict(hf_sd, strict=False)
    assert not missing, missing
    assert not unexpected, unexpected


def test_dinov2_matches_hf():
    from transformers import Dinov2Config as HC, Dinov2Model as HM

    from cornstarch_b200.models.vision_extra import Dinov2Config, Dinov2Model

    kw = dict(num_hidden_layers=2, hidden_size=32, num_attention_heads=4, image_size=28, patch_size=14)
    torch.manual_seed(0)
    hf = HM(HC(**kw)).eval()
    ours = Dinov2Model(Dinov2Config(**kw)).eval()
    _load(ours, hf.state_dict())
    px = torch.randn(2, 3, 28, 28)
    want = hf(pixel_values=px).last_hidden_state
    got = ours(pixel_values=px).last_hidden_state
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()
    assert Dinov2Model.module_names(ours.config) == ["embeddings", "encoder.layer.0", "encoder.layer.1", "layernorm"]


def test_pixtral_matches_hf():
    from transformers import PixtralVisionConfig as HC, PixtralVisionModel as HM

    from cornstarch_b200.models.vision_extra import PixtralVisionConfig, PixtralVisionModel

    kw = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=56, patch_size=14, head_dim=8)
    torch.manual_seed(0)
    hf = HM(HC(**kw)).eval()
    ours = PixtralVisionModel(PixtralVisionConfig(**kw)).eval()
    _load(ours, hf.state_dict())
    px = torch.randn(1, 3, 56, 42)
    want = hf(pixel_values=px, image_sizes=[(56, 42)]).last_hidden_state
    got = ours(pixel_values=px).last_hidden_state
    assert torch.allclose(got, want.view_as(got), atol=2e-3), (got - want.view_as(got)).abs().max()
    assert PixtralVisionModel.module_names(ours.config)[:4] == ["patch_conv", "ln_pre", "patch_positional_embedding", "transformer.layers.0"]


def test_qwen2_vision_matches_hf():
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig as HC
    from transformers.models.qwen2_vl.modeling_qwen2_vl import Qwen2VisionTransformerPretrainedModel as HM

    from cornstarch_b200.models.vision_extra import Qwen2VisionTransformerPretrainedModel, Qwen2VLVisionConfig

    kw = dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    torch.manual_seed(0)
    hf = HM(HC(**kw)).eval()
    ours = Qwen2VisionTransformerPretrainedModel(Qwen2VLVisionConfig(**kw)).eval()
    _load(ours, hf.state_dict())
    grid = torch.tensor([[1, 4, 6], [1, 4, 6]])
    x = torch.randn(48, 3 * 2 * 14 * 14)
    want = hf(x, grid_thw=grid)
    want = want if isinstance(want, torch.Tensor) else (want.pooler_output if getattr(want, "pooler_output", None) is not None else want[0])
    got = ours(hidden_states=x, grid_thw=grid).last_hidden_state
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()
    assert Qwen2VisionTransformerPretrainedModel.module_names(ours.config) == ["patch_embed", "rotary_pos_emb", "blocks.0", "blocks.1", "merger"]


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _mha(q, k, v, nh):
    B, S, H = q.shape
    sp = lambda t: t.view(B, S, nh, H // nh).transpose(1, 2)  # noqa: E731
    return F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(1, 2).reshape(B, S, H)


def test_intern_vit_block_math():
    from cornstarch_b200.models.vision_extra import InternVisionConfig, InternVisionModel

    torch.manual_seed(0)
    cfg = InternVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, image_size=28, patch_size=14)
    m = InternVisionModel(cfg).eval()
    px = torch.randn(2, 3, 28, 28)
    got = m(pixel_values=px).last_hidden_state
    L = m.encoder.layers[0]
    x = m.embeddings(px)
    h = _rms(x, L.norm1.weight, 1e-6)
    q, k, v = F.linear(h, L.attn.qkv.weight).split(32, dim=-1)
    q, k = _rms(q, L.attn.q_norm.weight, 1e-6), _rms(k, L.attn.k_norm.weight, 1e-6)
    x = x + F.linear(_mha(q, k, v, 4), L.attn.proj.weight, L.attn.proj.bias) * L.ls1
    h = _rms(x, L.norm2.weight, 1e-6)
    x = x + F.linear(F.gelu(F.linear(h, L.mlp.fc1.weight, L.mlp.fc1.bias)), L.mlp.fc2.weight, L.mlp.fc2.bias) * L.ls2
    assert torch.allclose(got, x, atol=1e-5)
    assert InternVisionModel.module_names(cfg) == ["embeddings", "encoder.layers.0"]


@pytest.mark.parametrize("post", [False, True])
def test_evaclip_block_math(post):
    from cornstarch_b200.models.vision_extra import EvaCLIPVisionConfig, EvaCLIPVisionModel

    torch.manual_seed(0)
    cfg = EvaCLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, image_size=28,
                              patch_size=14, use_rms_norm=True, k_bias=False, post_layernorm=post)
    m = EvaCLIPVisionModel(cfg).eval()
    px = torch.randn(2, 3, 28, 28)
    out = m(pixel_values=px)
    L = m.vision_model.encoder.layers[0]
    a = L.self_attn
    x = m.vision_model.embeddings(px)
    n1 = lambda t: _rms(t, L.layer_norm1.weight, 1e-5)  # noqa: E731
    n2 = lambda t: _rms(t, L.layer_norm2.weight, 1e-5)  # noqa: E731
    h = x if post else n1(x)
    o = F.linear(_mha(F.linear(h, a.q_proj.weight, a.q_proj.bias), F.linear(h, a.k_proj.weight), F.linear(h, a.v_proj.weight, a.v_proj.bias), 4),
                 a.out_proj.weight, a.out_proj.bias)
    x = x + (n1(o) if post else o)
    h = x if post else n2(x)
    mm = F.linear(F.gelu(F.linear(h, L.mlp.fc1.weight, L.mlp.fc1.bias)), L.mlp.fc2.weight, L.mlp.fc2.bias)
    x = x + (n2(mm) if post else mm)
    assert torch.allclose(out.last_hidden_state, x, atol=1e-5)
    assert EvaCLIPVisionModel.module_names(cfg) == ["vision_model.embeddings", "vision_model.encoder.layers.0", "vision_model.post_layernorm"]


def test_phi4_audio_matches_hf():
    from transformers.models.phi4_multimodal.configuration_phi4_multimodal import Phi4MultimodalAudioConfig as HC
    from transformers.models.phi4_multimodal.modeling_phi4_multimodal import Phi4MultimodalAudioModel as HM

    from cornstarch_b200.models.phi4_audio import Phi4MultimodalAudioConfig, Phi4MultimodalAudioModel

    kw = dict(hidden_size=32, intermediate_size=48, num_blocks=2, num_attention_heads=4, input_size=16, nemo_conv_channels=32,
              ext_pw_out_channel=32, kernel_size=3, time_reduction=8)
    torch.manual_seed(0)
    hf = HM(HC(depthwise_separable_out_channel=32, **kw)).eval()
    ours = Phi4MultimodalAudioModel(Phi4MultimodalAudioConfig(depthwise_separable_out_channel=32, **kw)).eval()
    _load(ours, hf.state_dict())
    x = torch.randn(2, 64, 16)
    want = hf(x, mask=None)
    want = want if isinstance(want, torch.Tensor) else want[0]
    got = ours(audio_input_features=x).last_hidden_state
    assert got.shape == want.shape, (got.shape, want.shape)
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()
    assert Phi4MultimodalAudioModel.module_names(ours.config) == ["encoder_embedding", "embed", "relative_attention_bias_layer",
                                                                    "encoders.0", "encoders.1"]
