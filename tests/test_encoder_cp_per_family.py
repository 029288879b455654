"""Context parallelism of the encoders per family (2 gloo ranks): tokens split uniformly after the embeddings, K/V gathered
for full attention; the gathered output equals the unsharded encoder's, and so does the gradient of the input."""

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed

FAMILIES = ["siglip", "clip", "vit", "dinov2", "evaclip", "pixtral", "whisper", "qwen2_audio", "phi4_audio", "internvit"]


def _features(model, kind, x):
    if kind == "phi4":
        out = model(audio_input_features=x)
    else:
        out = model(pixel_values=x) if kind.startswith("image") else model(input_features=x)
    return out["last_hidden_state"] if isinstance(out, dict) else out[0]


def _check(ref, model, kind, x, world, sp_mode="ring_attn"):
    from cornstarch_b200.parallel import comm
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    xr = x.clone().requires_grad_(True)
    want = _features(ref, kind, xr)
    wgt = torch.randn(want.shape, generator=torch.Generator().manual_seed(9))
    (want.float() * wgt).sum().backward()
    sc = ShardConfig(sequence_parallel_process_group=dist.group.WORLD, enable_sequence_parallelism=True,
                     sequence_parallelism_mode=sp_mode, enable_tensor_parallelism=False, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    xs = x.clone().requires_grad_(True)
    local = _features(model, kind, xs)
    assert local.shape[1] < want.shape[1], "the encoder did not split its tokens"
    full = comm.gather_forward_split_backward(local, 1, dist.group.WORLD)
    assert torch.allclose(full, want, atol=2e-4, rtol=1e-3), (full - want).abs().max()
    (full.float() * wgt).sum().backward()
    gx = xs.grad  # the split after the embeddings gathers the token gradients of all ranks in its backward pass
    err, ref_max = (gx - xr.grad).abs().max().item(), xr.grad.abs().max().item()
    assert ref_max > 0 and err <= 2e-3 * ref_max, (err, ref_max)


def _worker2(rank, world, family, sp_mode="ring_attn"):
    big = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=224, patch_size=14)
    from cornstarch_b200.models import vision as V
    from cornstarch_b200.models import vision_extra as X
    from cornstarch_b200.models import whisper as W

    def build():
        if family == "siglip":
            return V.SiglipVisionModel(V.SiglipVisionConfig(**big)), "image"
        if family == "clip":
            return V.CLIPVisionModel(V.CLIPVisionConfig(**big)), "image"
        if family == "vit":
            return V.ViTModel(V.ViTConfig(**big)), "image"
        if family == "dinov2":
            return X.Dinov2Model(X.Dinov2Config(**big)), "image"
        if family == "evaclip":
            return X.EvaCLIPVisionModel(X.EvaCLIPVisionConfig(**big)), "image"
        if family == "internvit":
            return X.InternVisionModel(X.InternVisionConfig(**big)), "image"  # q / k normalised over the full width, per token
        if family == "pixtral":
            return X.PixtralVisionModel(X.PixtralVisionConfig(**big, head_dim=16)), "image"
        if family == "phi4_audio":
            # the conformer's causal convolutions (kernel 3) need the two tokens before a rank's chunk; 65 tokens split 33 / 32
            from cornstarch_b200.models.phi4_audio import Phi4MultimodalAudioConfig, Phi4MultimodalAudioModel

            return Phi4MultimodalAudioModel(Phi4MultimodalAudioConfig(
                hidden_size=64, intermediate_size=96, num_blocks=2, num_attention_heads=4, input_size=16, nemo_conv_channels=32,
                ext_pw_out_channel=64, kernel_size=3, time_reduction=8, depthwise_separable_out_channel=64)), "phi4"
        cfg = dict(num_mel_bins=8, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, max_source_positions=300)
        if family == "whisper":
            return W.WhisperEncoder(W.WhisperConfig(**cfg)), "audio"
        return W.Qwen2AudioEncoder(W.Qwen2AudioEncoderConfig(**cfg)), "audio"

    torch.manual_seed(0)
    ref, kind = build()
    torch.manual_seed(0)
    model, _ = build()
    model.load_state_dict(ref.state_dict())
    g = torch.Generator().manual_seed(5)
    if kind == "phi4":
        x = torch.randn(2, 520 if sp_mode == "ring_attn" else 512, 16, generator=g)  # Ulysses wants equal shards
    else:
        x = torch.randn(2, 3, 224, 224, generator=g) if kind == "image" else torch.randn(2, 8, 600, generator=g)
    _check(ref, model, kind, x, world, sp_mode)


def _group_worker(rank, world, families):
    for family in families:
        try:
            _worker2(rank, world, family)
        except Exception as e:  # noqa: BLE001
            raise AssertionError(f"family {family}: {e}") from e
        dist.barrier()


@pytest.mark.parametrize("families", [FAMILIES[:4], FAMILIES[4:]], ids=["vision_a", "vision_b_and_audio"])
def test_encoder_ring_attn_matches_unsharded(families):
    run_distributed(_group_worker, 2, families)


def test_phi4_audio_ulysses_matches_unsharded():
    """Tokens split between the conformer's attention layers (halo for the causal convolutions), heads inside them."""
    run_distributed(_worker2, 2, "phi4_audio", "all_to_all")


def _qwen2_vl_worker(rank, world):
    """The Qwen2-VL tower splits every image's tokens in whole 2 x 2 merge groups and keeps the image dimension in its
    output; gathered along the token dimension it equals the unsharded tower's (flattened) output."""
    from cornstarch_b200.models import vision_extra as X
    from cornstarch_b200.parallel import comm
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    cfg = dict(depth=2, embed_dim=64, hidden_size=48, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)
    torch.manual_seed(0)
    ref = X.Qwen2VisionTransformerPretrainedModel(X.Qwen2VLVisionConfig(**cfg))
    torch.manual_seed(0)
    model = X.Qwen2VisionTransformerPretrainedModel(X.Qwen2VLVisionConfig(**cfg))
    model.load_state_dict(ref.state_dict())
    grid = torch.tensor([[1, 16, 16], [1, 16, 16]])
    x = torch.randn(2 * 256, 3 * 2 * 14 * 14, generator=torch.Generator().manual_seed(5))
    xr = x.clone().requires_grad_(True)
    want = ref(hidden_states=xr, grid_thw=grid).last_hidden_state  # [2 * 64, 48]
    wgt = torch.randn(want.shape, generator=torch.Generator().manual_seed(9))
    (want.float() * wgt).sum().backward()
    sc = ShardConfig(sequence_parallel_process_group=dist.group.WORLD, enable_sequence_parallelism=True,
                     sequence_parallelism_mode="ring_attn", enable_tensor_parallelism=False, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    xs = x.clone().requires_grad_(True)
    local = model(hidden_states=xs, grid_thw=grid).last_hidden_state
    assert local.shape == (2, 64 // world, 48), local.shape
    full = comm.gather_forward_split_backward(local, 1, dist.group.WORLD).reshape(want.shape)
    assert torch.allclose(full, want, atol=2e-4, rtol=1e-3), (full - want).abs().max()
    (full.float() * wgt).sum().backward()
    err, ref_max = (xs.grad - xr.grad).abs().max().item(), xr.grad.abs().max().item()
    assert err <= 2e-3 * ref_max, (err, ref_max)


def test_qwen2_vl_tower_ring_attn_matches_unsharded():
    run_distributed(_qwen2_vl_worker, 2)
