"""Token-sharded tensor parallelism (activations between the parallel blocks hold 1/tp of the token rows; the
column-parallel projections gather inside the GEMM, the row-parallel ones scatter inside the GEMM): on 2 gloo ranks the
loss, the input-embedding gradient and every parameter gradient equal the replicated-activation layout and the
unsharded model; a 2-stage pipeline hands the token shard from stage to stage."""

import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed

KW = dict(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
          num_key_value_heads=2, max_position_embeddings=64)


def _shard(model, seq_shard):
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    sc = ShardConfig(tensor_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=True,
                     tensor_parallel_sequence_sharding=seq_shard, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    return model


def _worker(rank, world, family):
    from cornstarch_b200.models import llama as L
    from cornstarch_b200.optim.fused_adamw import FusedAdamW

    cfg_cls = {"llama": L.LlamaConfig, "qwen3": L.Qwen3Config, "phi3": L.Phi3Config}[family]
    extra = dict(head_dim=16) if family == "qwen3" else {}
    torch.manual_seed(0)
    ref = L.DecoderForCausalLM(cfg_cls(**KW, **extra))
    models = {}
    for mode in (False, True):
        torch.manual_seed(0)
        m = L.DecoderForCausalLM(cfg_cls(**KW, **extra))
        m.load_state_dict(ref.state_dict())
        models[mode] = _shard(m, mode)
    x = torch.randint(0, 128, (2, 24), generator=torch.Generator().manual_seed(5))
    ref_loss = ref(input_ids=x, labels=x).loss
    ref_loss.backward()
    losses = {}
    for mode, m in models.items():
        opt = FusedAdamW(m.parameters(), lr=0.0)  # the optimizer adds the partial norm-weight gradients over the tp ranks
        out = m(input_ids=x, labels=x)
        out.loss.backward()
        opt._reduce_partial_grads()
        losses[mode] = out.loss.item()
        assert abs(out.loss.item() - ref_loss.item()) < 2e-4 * max(1.0, abs(ref_loss.item())), (family, mode, out.loss.item(), ref_loss.item())
    assert models[True].model._partial_marked is not None, "the token-sharded path did not run"
    a, b = dict(models[False].named_parameters()), dict(models[True].named_parameters())
    checked = 0
    for n, p in a.items():
        if p.grad is None:
            continue
        assert b[n].grad is not None, n
        assert torch.allclose(p.grad, b[n].grad, atol=3e-5, rtol=2e-3), (family, n, (p.grad - b[n].grad).abs().max())
        checked += 1
    assert checked > 10
    # replicated parameters (norm weights) equal the unsharded model's gradients
    rp = dict(ref.named_parameters())
    for n, p in b.items():
        if p.dim() == 1 and rp[n].shape == p.shape and "q_norm" not in n and "k_norm" not in n:
            assert torch.allclose(p.grad, rp[n].grad, atol=3e-5, rtol=2e-3), (family, n)


def test_token_sharded_tp_matches_replicated_tp_and_unsharded():
    for family in ("llama", "qwen3", "phi3"):
        run_distributed(_worker, 2, family)


def _uneven_worker(rank, world):
    """A token count that does not split evenly falls back to replicated activations."""
    from cornstarch_b200.models import llama as L

    torch.manual_seed(0)
    ref = L.DecoderForCausalLM(L.LlamaConfig(**KW))
    torch.manual_seed(0)
    m = L.DecoderForCausalLM(L.LlamaConfig(**KW))
    m.load_state_dict(ref.state_dict())
    _shard(m, True)
    x = torch.randint(0, 128, (1, 23), generator=torch.Generator().manual_seed(6))
    want = ref(input_ids=x, labels=x).loss
    got = m(input_ids=x, labels=x).loss
    assert abs(got.item() - want.item()) < 2e-4 * max(1.0, abs(want.item()))
    assert getattr(m.model, "_partial_marked", None) is None


def test_token_sharded_tp_falls_back_on_uneven_token_counts():
    run_distributed(_uneven_worker, 2)
