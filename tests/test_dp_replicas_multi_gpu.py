"""Data-parallel replicas stay bitwise identical: after optimizer steps every rank of a data-parallel group holds the
same parameters, including those whose gradients autograd leaves in ``.grad`` instead of the flat ``main_grad`` arena
(the patch convolution, position and class embeddings of a ViT; embedding lookups and q/k norm weights under tensor
parallelism).  Such gradients are folded into the arena BEFORE the data-parallel reduction; if they were folded after it
each replica would step with its own local gradient and drift apart silently."""

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_gpu_ranks

pytestmark = pytest.mark.gpu


def _assert_replicas_equal(params, group, what):
    flat = torch.cat([p.detach().reshape(-1).float() for p in params])
    ws = dist.get_world_size(group)
    everyone = [torch.empty_like(flat) for _ in range(ws)]
    dist.all_gather(everyone, flat, group=group)
    for r in range(1, ws):
        assert torch.equal(everyone[0], everyone[r]), (what, r, (everyone[0] - everyone[r]).abs().max().item())
    assert torch.isfinite(flat).all()


def _dp_vlm_worker(rank, world, overlap):
    from cornstarch_b200.bench_support import SingleDeviceTrainer
    from cornstarch_b200.ops import _native as nat

    dev = torch.device("cuda", rank)
    tr = SingleDeviceTrainer("tiny", 2, 1, dev, dp_group=dist.group.WORLD, lr=1e-2)
    tr.overlap_reduce = overlap
    stray = [n for n, p in tr.model.named_parameters() if "embeddings" in n]
    assert stray, "the ViT front-end parameters are what this test is about"
    before = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    for _ in range(3):
        loss = tr.step_device()
    assert torch.isfinite(loss)
    nat.check_status()
    _assert_replicas_equal(list(tr.model.parameters()), dist.group.WORLD, "dp replicas")
    moved = [n for n, p in tr.model.named_parameters() if not torch.equal(p.detach(), before[n])]
    assert any("embeddings" in n for n in moved), "the ViT embeddings must have been trained"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_dp2_vlm_replicas_identical_after_steps(overlap):
    run_gpu_ranks(_dp_vlm_worker, 2, overlap)


def _tp_dp_worker(rank, world):
    """tp 2 x dp 2 of a Qwen3-style decoder (q_norm / k_norm weights see a tensor-parallel gradient reduction, the
    vocab-parallel embedding runs through F.embedding): replicas along dp are identical after the steps."""
    from cornstarch_b200.models.llama import DecoderForCausalLM, Qwen3Config
    from cornstarch_b200.ops import _native as nat
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.parallel.mesh import MultiModalProcessGroupMesh  # noqa: F401  (mesh code path stays importable)
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    tp_ranks = [[0, 1], [2, 3]]
    dp_ranks = [[0, 2], [1, 3]]
    tp_groups = [dist.new_group(r) for r in tp_ranks]
    dp_groups = [dist.new_group(r) for r in dp_ranks]
    tp_group = tp_groups[rank // 2]
    dp_group = dp_groups[rank % 2]
    torch.manual_seed(0)
    cfg = Qwen3Config(vocab_size=1000, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=64, max_position_embeddings=256, tie_word_embeddings=True)
    model = DecoderForCausalLM(cfg).cuda().bfloat16()
    sc = ShardConfig(tensor_parallel_process_group=tp_group, enable_tensor_parallelism=True)
    model, _ = ShardFormer(sc).optimize(model)
    assert model.lm_head.weight is model.model.embed_tokens.weight, "the tie must survive tensor parallelism"
    model.train()
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-2, max_norm=1.0, dp_group=dp_group, norm_groups=[tp_group])
    ids = torch.randint(0, 1000, (2, 256), generator=torch.Generator().manual_seed(100 + rank // 2)).cuda()  # same data inside a tp group
    dist.barrier()
    for _ in range(2):
        model(input_ids=ids, labels=ids).loss.backward()
        assert opt.reduce_dp_grads()
        opt.step()
        opt.zero_grad()
    nat.check_status()
    _assert_replicas_equal(list(model.parameters()), dp_group, "dp replicas of a tp shard")


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_tp2_dp2_replicas_identical_after_steps():
    run_gpu_ranks(_tp_dp_worker, 4)
