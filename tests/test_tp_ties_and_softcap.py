"""Tensor parallelism keeps two model-level properties of the unsharded model (2 gloo ranks):

* ``tie_word_embeddings``: after sharding, ``lm_head.weight`` is still the SAME Parameter as ``embed_tokens.weight``
  (each rank holds one shard of the tied matrix), and the loss and the tied gradient equal the unsharded model's;
* Gemma-2's final-logit soft-capping: the loss of the sharded model equals the unsharded one (the capped logits are
  gathered over the vocabulary shards before the cross-entropy), also under ring-attention context parallelism.
"""

import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed

KW = dict(vocab_size=200, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
          num_key_value_heads=2, max_position_embeddings=64)


def _shard(model, **kw):
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    sc = ShardConfig(extra_kwargs={"device": "cpu"}, **kw)
    ShardFormer(sc).optimize(model)
    return model


def _tied_worker(rank, world):
    from cornstarch_b200.models import llama as L

    torch.manual_seed(0)
    ref = L.DecoderForCausalLM(L.LlamaConfig(**KW, tie_word_embeddings=True))
    assert ref.lm_head.weight is ref.model.embed_tokens.weight
    torch.manual_seed(0)
    model = L.DecoderForCausalLM(L.LlamaConfig(**KW, tie_word_embeddings=True))
    model.load_state_dict(ref.state_dict())
    x = torch.randint(0, 200, (2, 24), generator=torch.Generator().manual_seed(3))
    ref_loss = ref(input_ids=x, labels=x).loss
    ref_loss.backward()
    _shard(model, tensor_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=True)
    assert model.lm_head.weight is model.model.embed_tokens.weight, "the tie was lost by the tensor-parallel layers"
    assert len({id(p) for p in model.parameters()}) == len(list(model.parameters()))
    loss = model(input_ids=x, labels=x).loss
    assert abs(loss.item() - ref_loss.item()) < 2e-4 * max(1.0, abs(ref_loss.item())), (loss.item(), ref_loss.item())
    loss.backward()
    w = model.lm_head.weight
    local = w.shape[0]
    lo = rank * local
    want = torch.zeros_like(w)
    hi = min(lo + local, ref.lm_head.weight.shape[0])
    if hi > lo:
        want[: hi - lo] = ref.lm_head.weight.grad[lo:hi]
    assert torch.allclose(w.grad, want, atol=2e-5, rtol=2e-3), (w.grad - want).abs().max()


def test_tied_embeddings_stay_tied_under_tp2():
    run_distributed(_tied_worker, 2)


def _softcap_worker(rank, world, mode):
    from cornstarch_b200.models import llama as L

    cfg = dict(**KW, head_dim=16, query_pre_attn_scalar=16, final_logit_softcapping=5.0)
    torch.manual_seed(0)
    ref = L.DecoderForCausalLM(L.Gemma2Config(**cfg))
    assert ref.model.spec.final_softcap == 5.0
    torch.manual_seed(0)
    model = L.DecoderForCausalLM(L.Gemma2Config(**cfg))
    model.load_state_dict(ref.state_dict())
    x = torch.randint(0, 200, (2, 32), generator=torch.Generator().manual_seed(4))  # labels reach beyond one shard's rows
    ref_loss = ref(input_ids=x, labels=x).loss
    if mode == "tp":
        _shard(model, tensor_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=True)
    else:
        _shard(model, sequence_parallel_process_group=dist.group.WORLD, enable_tensor_parallelism=False,
               sequence_parallelism_mode="ring_attn", context_parallel_distribution_mode="uniform")
    out = model(input_ids=x, labels=x)
    if mode == "tp":
        loss = out.loss
    else:
        # every context-parallel rank returns sp * (its share of the loss sum) / (global count): the mean over ranks is the loss
        t = out.loss.detach().clone()
        dist.all_reduce(t)
        loss = t / world
    assert abs(loss.item() - ref_loss.item()) < 2e-4 * max(1.0, abs(ref_loss.item())), (mode, loss.item(), ref_loss.item())
    out.loss.backward()


def test_gemma2_softcap_loss_under_tp2():
    run_distributed(_softcap_worker, 2, "tp")


def test_gemma2_softcap_loss_under_ring_attention():
    run_distributed(_softcap_worker, 2, "cp")
