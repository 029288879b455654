"""The reference-style layer names (``Linear1D_Col`` ...) built from plain PyTorch modules, and lazy construction."""

import torch
import torch.nn as nn

from cornstarch_b200.shardformer import layers as L


def test_from_native_module_without_group_keeps_the_function():
    torch.manual_seed(0)
    lin = nn.Linear(32, 48)
    x = torch.randn(3, 5, 32)
    for cls in (L.Linear1D_Col, L.Linear1D_Row):
        assert torch.allclose(cls.from_native_module(lin, None)(x), lin(x), atol=1e-5)
    fused = L.FusedLinear1D_Col.from_native_module(lin, None, split_sizes=[16, 16, 16])
    assert torch.allclose(fused(x), lin(x), atol=1e-5)

    emb = nn.Embedding(100, 32)
    ids = torch.randint(0, 100, (2, 7))
    pe = L.PaddingEmbedding.from_native_module(emb, None, make_vocab_size_divisible_by=64)
    assert pe.weight.shape[0] == 128 and torch.equal(pe(ids), emb(ids))
    ve = L.VocabParallelEmbedding1D.from_native_module(emb, None)
    assert torch.equal(ve(ids), emb(ids))

    head = nn.Linear(32, 100, bias=False)
    ph = L.PaddingLMHead.from_native_module(head, None, make_vocab_size_divisible_by=64)
    out = ph(x)
    assert out.shape[-1] == 128 and torch.allclose(out[..., :100], head(x), atol=1e-5) and out[..., 100:].abs().max() == 0
    vh = L.VocabParallelLMHead1D.from_native_module(head, None)
    assert vh.num_embeddings == 100

    ln = nn.LayerNorm(32)
    assert torch.allclose(L.FusedLayerNorm.from_native_module(ln)(x), ln(x), atol=1e-5)
    rms = nn.RMSNorm(32, eps=1e-6)
    assert torch.allclose(L.FusedRMSNorm.from_native_module(rms)(x), rms(x), atol=1e-5)
    assert L.DropoutForReplicatedInput(0.0)(x) is not None


def test_lazy_init_context_materialises_later():
    from cornstarch_b200.models.llama import LlamaConfig, LlamaForCausalLM

    with L.LazyInitContext():
        model = LlamaForCausalLM(LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2,
                                             num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=32))
    assert all(p.device.type == "meta" for p in model.parameters())
    L.LazyInitContext.materialize(model, device="cpu", dtype=torch.float32)
    assert all(p.device.type == "cpu" for p in model.parameters())
    ids = torch.randint(0, 64, (1, 8))
    assert torch.isfinite(model(input_ids=ids, labels=ids).loss)
