"""Tensor parallelism per model family (2 gloo ranks): the model sharded by its policy gives the loss / output of the
unsharded model with the same weights, the same gradient with respect to its input, and the same gradients for the
parameters that stay replicated (norm weights).  The reference runs this grid in tests/test_shardformer/test_hybrid_parallel.py."""

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed

KW = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
          num_key_value_heads=2, max_position_embeddings=64)


def _build(family):
    from cornstarch_b200.models import llama as L
    from cornstarch_b200.models import moe as M
    from cornstarch_b200.models import text_legacy as T
    from cornstarch_b200.models import vision as V
    from cornstarch_b200.models import vision_extra as X
    from cornstarch_b200.models import whisper as W

    vis = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    if family in ("llama", "mistral", "qwen2", "qwen3", "gemma", "phi3"):
        cfg_cls = {"llama": L.LlamaConfig, "mistral": L.MistralConfig, "qwen2": L.Qwen2Config, "qwen3": L.Qwen3Config,
                   "gemma": L.GemmaConfig, "phi3": L.Phi3Config}[family]
        extra = dict(head_dim=16) if family in ("qwen3", "gemma") else {}
        return L.DecoderForCausalLM(cfg_cls(**KW, **extra)), "text"
    if family == "gemma2":
        return L.DecoderForCausalLM(L.Gemma2Config(**KW, head_dim=16, query_pre_attn_scalar=16)), "text"
    if family == "mixtral":
        return M.MoeForCausalLM(M.MixtralConfig(**KW, num_local_experts=4, num_experts_per_tok=2)), "text"
    if family == "gpt2":
        return T.GPT2LMHeadModel(T.GPT2Config(n_layer=2, n_embd=64, n_head=4, vocab_size=128, n_positions=64, tie_word_embeddings=False)), "text"
    if family == "opt":
        return T.OPTForCausalLM(T.OPTConfig(vocab_size=128, hidden_size=64, ffn_dim=128, num_hidden_layers=2, num_attention_heads=4,
                                            max_position_embeddings=64, word_embed_proj_dim=64, tie_word_embeddings=False)), "text"
    if family == "bert":
        return T.BertForMaskedLM(T.BertConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                              num_attention_heads=4, max_position_embeddings=64, tie_word_embeddings=False)), "text"
    if family == "siglip":
        return V.SiglipVisionModel(V.SiglipVisionConfig(**vis)), "image"
    if family == "clip":
        return V.CLIPVisionModel(V.CLIPVisionConfig(**vis)), "image"
    if family == "vit":
        return V.ViTModel(V.ViTConfig(**vis)), "image"
    if family == "dinov2":
        return X.Dinov2Model(X.Dinov2Config(**vis)), "image"
    if family == "whisper":
        return W.WhisperEncoder(W.WhisperConfig(num_mel_bins=8, d_model=64, encoder_layers=2, encoder_attention_heads=4,
                                                encoder_ffn_dim=128, max_source_positions=10)), "audio"
    if family == "gemma3":
        return L.DecoderForCausalLM(L.Gemma3TextConfig(**KW, head_dim=16, query_pre_attn_scalar=16,
                                                       layer_types=["sliding_attention", "full_attention"])), "text"
    if family == "qwen3_moe":
        return M.MoeForCausalLM(M.Qwen3MoeConfig(**KW, head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32)), "text"
    if family == "llama4":
        from cornstarch_b200.models.llama4 import Llama4ForCausalLM, Llama4TextConfig

        return Llama4ForCausalLM(Llama4TextConfig(vocab_size=128, hidden_size=64, intermediate_size=48, intermediate_size_mlp=128,
                                                  num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                                                  num_local_experts=4, num_experts_per_tok=1, interleave_moe_layer_step=2,
                                                  max_position_embeddings=64, attention_chunk_size=64)), "text"
    if family == "internvit":
        return X.InternVisionModel(X.InternVisionConfig(**vis, qk_normalization=False)), "image"
    if family == "evaclip":
        return X.EvaCLIPVisionModel(X.EvaCLIPVisionConfig(**vis)), "image"
    if family == "pixtral":
        return X.PixtralVisionModel(X.PixtralVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                                                          num_attention_heads=4, image_size=56, patch_size=14, head_dim=16)), "image56"
    if family == "phi4_audio":
        from cornstarch_b200.models.phi4_audio import Phi4MultimodalAudioConfig, Phi4MultimodalAudioModel

        return Phi4MultimodalAudioModel(Phi4MultimodalAudioConfig(
            hidden_size=64, intermediate_size=96, num_blocks=2, num_attention_heads=4, input_size=16, nemo_conv_channels=32,
            ext_pw_out_channel=64, kernel_size=3, time_reduction=8, depthwise_separable_out_channel=64)), "phi4"
    if family == "qwen2_vl":
        return X.Qwen2VisionTransformerPretrainedModel(X.Qwen2VLVisionConfig(
            depth=2, embed_dim=64, hidden_size=48, num_heads=4, mlp_ratio=2, patch_size=14, spatial_merge_size=2, temporal_patch_size=2)), "qwen2vl"
    if family == "qwen2_audio":
        return W.Qwen2AudioEncoder(W.Qwen2AudioEncoderConfig(num_mel_bins=8, d_model=64, encoder_layers=2, encoder_attention_heads=4,
                                                             encoder_ffn_dim=128, max_source_positions=10)), "audio"
    raise KeyError(family)


def _run(model, kind, x):
    if kind == "text":
        out = model(input_ids=x, labels=x)
        return out.loss
    if kind == "phi4":
        out = model(audio_input_features=x)
    elif kind == "qwen2vl":
        out = model(hidden_states=x, grid_thw=torch.tensor([[1, 4, 4], [1, 4, 4]]))
    elif kind in ("image", "image56"):
        out = model(pixel_values=x)
    else:
        out = model(input_features=x)
    h = out["last_hidden_state"] if isinstance(out, dict) else out[0]
    return h.float().square().mean()


def _worker(rank, world, family):
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    torch.manual_seed(0)
    ref, kind = _build(family)
    torch.manual_seed(0)
    model, _ = _build(family)
    model.load_state_dict(ref.state_dict())
    g = torch.Generator().manual_seed(5)
    if kind == "text":
        x = torch.randint(0, 128, (2, 24), generator=g)
    elif kind == "image":
        x = torch.randn(2, 3, 28, 28, generator=g, requires_grad=True)
    elif kind == "image56":
        x = torch.randn(2, 3, 56, 56, generator=g, requires_grad=True)
    elif kind == "phi4":
        x = torch.randn(2, 64, 16, generator=g, requires_grad=True)
    elif kind == "qwen2vl":
        x = torch.randn(32, 3 * 2 * 14 * 14, generator=g, requires_grad=True)
    else:
        x = torch.randn(2, 8, 20, generator=g, requires_grad=True)
    xr = x.detach().clone().requires_grad_(x.requires_grad) if x.is_floating_point() else x
    ref_loss = _run(ref, kind, xr)
    ref_loss.backward()

    sc = ShardConfig(tensor_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=True, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    n_local = sum(p.numel() for p in model.parameters())
    n_full = sum(p.numel() for p in ref.parameters())
    assert n_local < n_full, "the policy sharded nothing"
    loss = _run(model, kind, x)
    assert abs(loss.item() - ref_loss.item()) < 2e-4 * max(1.0, abs(ref_loss.item())), (family, loss.item(), ref_loss.item())
    loss.backward()
    if x.is_floating_point():
        assert torch.allclose(x.grad, xr.grad, atol=5e-5, rtol=1e-3), (x.grad - xr.grad).abs().max()
    checked = 0
    ref_params = dict(ref.named_parameters())
    for n, p in model.named_parameters():
        rp = ref_params.get(n)
        if rp is None or rp.shape != p.shape or p.grad is None or rp.grad is None or p.dim() != 1 or "bias" in n:
            continue
        assert torch.allclose(p.grad, rp.grad, atol=2e-5, rtol=2e-3), (family, n, (p.grad - rp.grad).abs().max())
        checked += 1
    assert checked > 0


GROUPS = {
    "dense_decoders": ["llama", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "gemma3", "phi3"],
    "moe_and_legacy": ["mixtral", "qwen3_moe", "llama4", "gpt2", "opt", "bert"],
    "vision": ["siglip", "clip", "vit", "dinov2", "internvit", "evaclip", "pixtral", "qwen2_vl"],
    "audio": ["whisper", "qwen2_audio", "phi4_audio"],
}


def _group_worker(rank, world, families):
    for family in families:  # one process group for the whole list: starting ranks costs more than the checks
        try:
            _worker(rank, world, family)
        except Exception as e:  # noqa: BLE001
            raise AssertionError(f"family {family}: {e}") from e
        dist.barrier()


@pytest.mark.parametrize("group", sorted(GROUPS))
def test_tp2_matches_unsharded(group):
    run_distributed(_group_worker, 2, GROUPS[group])


def _gather_worker(rank, world, family):
    """Checkpoint view of a tensor-parallel model: every sharded parameter gathers back to the unsharded tensor, and the
    unsharded tensor shards to what the rank holds."""
    from cornstarch_b200.plugin.checkpoint_io import _tp_info, gather_full_tensor, shard_full_tensor
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    torch.manual_seed(0)
    ref, _ = _build(family)
    torch.manual_seed(0)
    model, _ = _build(family)
    model.load_state_dict(ref.state_dict())
    sc = ShardConfig(tensor_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=True, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    info = _tp_info(model)
    assert info, "no tensor-parallel parameter found"
    full = dict(ref.named_parameters())
    for name, p in model.named_parameters():
        if name not in info:
            continue
        back = gather_full_tensor(name, p.data, info, dist.group.WORLD)
        assert back.shape == full[name].shape and torch.equal(back, full[name].data), name
        assert torch.equal(shard_full_tensor(name, full[name].data, info, dist.group.WORLD), p.data), name


def _gather_group_worker(rank, world, families):
    for family in families:
        _gather_worker(rank, world, family)
        dist.barrier()


def test_tp_parameters_gather_to_unsharded():
    run_distributed(_gather_group_worker, 2, ["llama", "phi3", "gpt2", "mixtral", "siglip"])
