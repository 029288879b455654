"""Expert parallelism: dispatch / combine all-to-all with experts sharded over ranks equals the local MoE block."""

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _worker(rank, world, num_experts):
    from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
    from cornstarch_b200.parallel.ep import shard_experts

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=num_experts, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MixtralSparseMoeBlock(cfg)
    torch.manual_seed(0)
    sharded = MixtralSparseMoeBlock(cfg)
    expert_params = shard_experts(sharded, dist.group.WORLD)
    assert len(sharded.experts) == num_experts // world and all(p.expert_parallel for p in expert_params)
    # every rank has its own tokens (data parallel over the same group)
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(2, 9 + rank, 32, generator=g)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, la = full(xa)
    yb, lb = sharded(xb)
    assert torch.allclose(ya, yb, atol=1e-5), (ya - yb).abs().max()
    assert torch.allclose(la, lb)
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
    assert torch.allclose(full.gate.weight.grad, sharded.gate.weight.grad, atol=1e-5)
    # expert weights: the sharded gradient holds contributions of ALL ranks' tokens, the local block only mine
    per = num_experts // world
    zero = torch.zeros_like(full.experts[0].w1.weight)
    mine = torch.stack([e.w1.weight.grad if e.w1.weight.grad is not None else zero for e in full.experts])
    everyone = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    total = sum(everyone)
    for j in range(per):
        got = sharded.experts[j].w1.weight.grad
        assert torch.allclose(got, total[rank * per + j], atol=1e-4), (rank, j, (got - total[rank * per + j]).abs().max())


def test_ep2_four_experts():
    run_distributed(_worker, 2, 4)


def test_ep4_four_experts():
    run_distributed(_worker, 4, 4)


def test_regroup_permutation_and_counts_without_host_values():
    """The device-side helpers of the dispatch: pairs per expert, and the permutation from (source, local expert) to
    (local expert, source) order, against their plain statements (segments of length zero included)."""
    from cornstarch_b200.parallel.ep import by_expert_order, expert_counts

    flat_e = torch.tensor([3, 0, 3, 1, 0, 3])
    assert expert_counts(flat_e, 5).tolist() == [2, 1, 0, 3, 0]
    rc = [[2, 0, 1], [0, 3, 1], [1, 1, 0]]  # [source][local expert]
    ws, local = 3, 3
    starts, pos = [], 0
    for s in range(ws):
        for e in range(local):
            starts.append(pos)
            pos += rc[s][e]
    want = [i for e in range(local) for s in range(ws) for i in range(starts[s * local + e], starts[s * local + e] + rc[s][e])]
    assert by_expert_order(torch.tensor(rc), pos).tolist() == want


def test_capacity_mode_in_one_process_without_a_group():
    """``set_expert_capacity``: the static-shape form with every expert local, no torch.distributed at all."""
    from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
    from cornstarch_b200.parallel.ep import dropped_pairs, set_expert_capacity

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MixtralSparseMoeBlock(cfg)
    torch.manual_seed(0)
    capped = MixtralSparseMoeBlock(cfg)
    set_expert_capacity(capped, 4.0)  # room for every pair
    assert len(capped.experts) == 4 and not dist.is_initialized()
    x = torch.randn(2, 12, 32)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, _ = full(xa)
    yb, _ = capped(xb)
    assert int(dropped_pairs(capped)) == 0
    assert torch.allclose(ya, yb, atol=1e-5)
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
    for ea, eb in zip(full.experts, capped.experts):
        ga, gb = ea.w1.weight.grad, eb.w1.weight.grad
        assert torch.allclose(torch.zeros_like(gb) if ga is None else ga, gb, atol=1e-5)
    set_expert_capacity(capped, 0.5)  # too little room: pairs are dropped and counted
    capped(x)
    assert int(dropped_pairs(capped)) > 0


def _capacity_worker(rank, world, factor):
    """Static-shape (capacity) dispatch: with room for every pair it equals the local MoE block exactly, in outputs and in
    every gradient; with too little room the surplus pairs are dropped, counted, and contribute nothing."""
    from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
    from cornstarch_b200.parallel.ep import shard_experts

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MixtralSparseMoeBlock(cfg)
    torch.manual_seed(0)
    sharded = MixtralSparseMoeBlock(cfg)
    shard_experts(sharded, dist.group.WORLD, capacity_factor=factor)
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(2, 12, 32, generator=g)  # equal token counts on every rank: the shapes of the exchange are static
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, _ = full(xa)
    yb, _ = sharded(xb)
    dropped = int(sharded.ep.dropped_pairs)
    from cornstarch_b200.parallel.ep import dropped_pairs

    assert int(dropped_pairs(sharded)) == dropped and dropped_pairs(full) is None
    if factor >= 4.0:  # capacity = every pair of the rank: nothing can be dropped
        assert dropped == 0
        assert torch.allclose(ya, yb, atol=1e-5), (ya - yb).abs().max()
        ya.square().sum().backward()
        yb.square().sum().backward()
        assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
        assert torch.allclose(full.gate.weight.grad, sharded.gate.weight.grad, atol=1e-5)
        per = 4 // world
        zero = torch.zeros_like(full.experts[0].w1.weight)
        mine = torch.stack([e.w1.weight.grad if e.w1.weight.grad is not None else zero for e in full.experts])
        everyone = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        total = sum(everyone)
        for j in range(per):
            assert torch.allclose(sharded.experts[j].w1.weight.grad, total[rank * per + j], atol=1e-4)
    else:
        assert dropped > 0
        assert torch.isfinite(yb).all()
        yb.square().sum().backward()
        assert torch.isfinite(xb.grad).all()
        # a token whose pairs were all kept is computed exactly
        same = (ya - yb).abs().amax(dim=-1) < 1e-5
        assert same.any() and not same.all()


def test_ep2_capacity_mode_is_exact_with_room_for_every_pair():
    run_distributed(_capacity_worker, 2, 4.0)


def test_ep2_capacity_mode_drops_and_counts_the_surplus():
    run_distributed(_capacity_worker, 2, 0.5)


def _capacity_gpu_worker(rank, world):
    from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
    from cornstarch_b200.parallel.ep import shard_experts

    cfg = MixtralConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MixtralSparseMoeBlock(cfg).cuda().bfloat16()
    torch.manual_seed(0)
    sharded = MixtralSparseMoeBlock(cfg).cuda().bfloat16()
    shard_experts(sharded, dist.group.WORLD, capacity_factor=4.0)  # room for every pair: nothing dropped
    x = torch.randn(2, 384, 256, generator=torch.Generator().manual_seed(3)).cuda().bfloat16()
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, _ = full(xa)
    yb, _ = sharded(xb)
    ya.float().square().sum().backward()
    yb.float().square().sum().backward()
    assert int(sharded.ep.dropped_pairs) == 0
    for name, a, b in (("y", yb, ya), ("dx", xb.grad, xa.grad), ("dgate", sharded.gate.weight.grad, full.gate.weight.grad),
                       ("dw1", sharded.experts[1].w1.weight.grad, full.experts[1].w1.weight.grad)):
        err = (a.float() - b.float()).abs().max().item()
        assert err <= 2e-2 * max(1.0, b.float().abs().max().item()), (name, err)


@pytest.mark.gpu
def test_capacity_mode_on_the_device_equals_the_local_block():
    from tests.dist_utils import run_gpu_ranks

    run_gpu_ranks(_capacity_gpu_worker, 1)


def _unequal_tokens_worker(rank, world):
    """Capacity mode with a fixed ``capacity_tokens``: ranks with different numbers of tokens exchange buffers of one shape,
    and with room for every pair the result is the local block's."""
    from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
    from cornstarch_b200.parallel.ep import shard_experts

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MixtralSparseMoeBlock(cfg)
    torch.manual_seed(0)
    sharded = MixtralSparseMoeBlock(cfg)
    shard_experts(sharded, dist.group.WORLD, capacity_factor=4.0, capacity_tokens=32)
    x = torch.randn(2, 9 + 5 * rank, 32, generator=torch.Generator().manual_seed(10 + rank))  # 18 and 28 tokens
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya, _ = full(xa)
    yb, _ = sharded(xb)
    assert int(sharded.ep.dropped_pairs) == 0
    assert torch.allclose(ya, yb, atol=1e-5), (ya - yb).abs().max()
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)


def test_ep2_capacity_mode_with_unequal_token_counts():
    run_distributed(_unequal_tokens_worker, 2)


def _ckpt_worker(rank, world):
    from cornstarch_b200.models.moe import MixtralConfig, MoeForCausalLM
    from cornstarch_b200.parallel.ep import gather_full_state_dict, shard_experts

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    full = MoeForCausalLM(cfg)
    torch.manual_seed(0)
    sharded = MoeForCausalLM(cfg)
    shard_experts(sharded, dist.group.WORLD)
    # the sharded model names its experts globally and reassembles to the unsharded state dict
    names = [k for k in sharded.state_dict() if ".experts." in k]
    per = 4 // world
    assert all(int(k.split(".experts.")[1].split(".")[0]) in range(rank * per, (rank + 1) * per) for k in names)
    sd = gather_full_state_dict(sharded, dist.group.WORLD)
    if rank == 0:
        ref = full.state_dict()
        assert set(sd) == set(ref)
        assert all(torch.equal(sd[k], ref[k]) for k in ref)
    # loading a full state dict into a sharded model keeps only the local experts
    torch.manual_seed(1)
    other = MoeForCausalLM(cfg)
    missing, unexpected = sharded.load_state_dict(other.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    e = rank * per
    assert torch.equal(sharded.model.layers[1].block_sparse_moe.experts[0].w1.weight, other.model.layers[1].block_sparse_moe.experts[e].w1.weight)


def test_expert_sharded_state_dict_round_trip():
    run_distributed(_ckpt_worker, 2)


def _zero_state_worker(rank, world):
    """ZeRO-1 optimizer state: every rank holds a slice of the flat state; the gathered view is whole on every rank and
    loading a whole per-parameter state fills exactly the local slice - also for a parameter that straddles the boundary."""
    from cornstarch_b200.optim.fused_adamw import _Region

    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(n).bfloat16()) for n in (192, 64, 320)]  # 576 elements: the cut at 288 is inside the last one
    for split in (False, True):
        region = _Region([torch.nn.Parameter(p.data.clone()) for p in params], torch.bfloat16, (rank, world), None, split_master=split)
        assert region.hi - region.lo == region.numel // world
        whole = {k: torch.randn(region.numel, generator=torch.Generator().manual_seed(5 + i))
                 for i, k in enumerate(("master", "exp_avg", "exp_avg_sq"))}
        for p, off in zip(region.params, region.offsets):
            region.import_param_state(off, p.numel(), {k: v[off : off + p.numel()] for k, v in whole.items()})
        got = region.gathered_states(dist.group.WORLD)
        covered = torch.zeros(region.numel, dtype=torch.bool)
        for p, off in zip(region.params, region.offsets):
            covered[off : off + p.numel()] = True
        for k in whole:
            assert torch.equal(got[k][covered], whole[k][covered]), (split, k)
        # the local slice holds exactly its part
        assert torch.equal(region.exp_avg, whole["exp_avg"][region.lo : region.hi].where(covered[region.lo : region.hi], region.exp_avg))


def test_zero1_state_gathers_whole_and_loads_by_overlap():
    run_distributed(_zero_state_worker, 2)


def _tp_ep_worker(rank, world, capacity):
    """Language model only, tensor parallel 2 inside every expert AND the experts sharded over 2 data-parallel replicas:
    each replica's loss equals the single-process model's on the same samples, and an optimizer step goes through."""
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.models.moe import MixtralConfig, MoeForCausalLM
    from cornstarch_b200.multimodal import MultimodalModel
    from cornstarch_b200.optim.fused_adamw import FusedAdamW
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin

    cfg = MixtralConfig(vocab_size=512, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2, max_position_embeddings=256)
    torch.manual_seed(0)
    ref = MoeForCausalLM(cfg)
    torch.manual_seed(0)
    llm = MoeForCausalLM(cfg)
    ids = torch.randint(0, 512, (4, 64), generator=torch.Generator().manual_seed(1))
    ref_losses = [ref(input_ids=ids[i : i + 1], labels=ids[i : i + 1]).loss.item() for i in range(4)]
    model = MultimodalModel(encoders={}, language_model=llm)
    plugin = MultimodalParallelPlugin(
        encoder_plugins={},
        language_model_plugin=ModalParallelPlugin(tp_size=2, pipeline_template=PipelineTemplate.even_split(llm, 1), ep_size=2,
                                                  ep_capacity_factor=capacity),
        precision=None, num_microbatches=2, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    model, opt, criterion, *_ = booster.boost(model, FusedAdamW, criterion=lambda out, batch: out.loss)
    replica = plugin.pg_mesh.coords[0][plugin.pg_mesh.dp_axis]
    mine = ids[replica * 2 : (replica + 1) * 2]
    out = booster.execute_pipeline(iter([{"input_ids": mine, "labels": mine}]), model, criterion, opt, return_loss=True)
    want = sum(ref_losses[replica * 2 : (replica + 1) * 2]) / 2
    assert abs(out["loss"].item() - want) < 1e-4, (out["loss"].item(), want)
    opt.step()
    opt.zero_grad()


def test_plugin_tensor_parallel_experts_sharded_over_replicas():
    run_distributed(_tp_ep_worker, 4, None)  # (with a capacity factor the tensor-parallel experts run the same loop)


def _shardformer_worker(rank, world):
    """``ShardConfig(expert_parallel_process_group=...)``: ShardFormer shards the experts of a MoE decoder by itself."""
    from cornstarch_b200.models.moe import MixtralConfig, MoeForCausalLM
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    cfg = MixtralConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, num_local_experts=4, num_experts_per_tok=2)
    torch.manual_seed(0)
    ref = MoeForCausalLM(cfg)
    torch.manual_seed(0)
    model = MoeForCausalLM(cfg)
    sc = ShardConfig(enable_tensor_parallelism=False, expert_parallel_process_group=dist.group.WORLD)
    ShardFormer(sc).optimize(model)
    blocks = [m for m in model.modules() if getattr(m, "ep", None) is not None]
    assert len(blocks) == 2 and all(len(b.experts) == 2 for b in blocks)
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(rank))
    want = ref(input_ids=ids, labels=ids).loss
    got = model(input_ids=ids, labels=ids).loss
    assert abs(want.item() - got.item()) < 1e-5


def test_shardformer_shards_experts_over_the_configured_group():
    run_distributed(_shardformer_worker, 2)
