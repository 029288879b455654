"""Heterogeneous (Oobleck-style) pipelines: mesh table, batch sampler, and training parity of two pipelines with
different stage counts and micro-batch counts against the single-process model."""

import numpy as np
import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _tpl(stages_layers):
    from cornstarch_b200.pipeline_template import PipelineTemplate

    mods, k = [], 0
    for n in stages_layers:
        mods.append([f"layers.{k + i}" for i in range(n)])
        k += n
    return PipelineTemplate("m", mods)


def test_mesh_table_matches_reference_docstring():
    from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousProcessGroupMesh as Mesh

    m = Mesh([_tpl([2, 2, 2]), _tpl([3, 3]), _tpl([3, 3])], tp_size=2, rank=8)
    expected = [[[0, 1], [0, 1], [2, 3], [2, 3], [4, 5], [4, 5]],
                [[6, 7], [6, 7], [6, 7], [8, 9], [8, 9], [8, 9]],
                [[10, 11], [10, 11], [10, 11], [12, 13], [12, 13], [12, 13]]]
    assert np.array_equal(m.mesh, np.array(expected))
    assert m.unit_dp_ranks(2, 0) == (2, 6, 10) and m.unit_dp_ranks(5, 1) == (5, 9, 13)
    assert m.coords[0] == (1, 3, 0)


def test_batch_sampler_example():
    from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousBatchSampler as S

    a = list(S(range(20), pipeline_index=0, microbatch_size=2, num_microbatches=[2, 3], shuffle=False))
    b = list(S(range(20), pipeline_index=1, microbatch_size=2, num_microbatches=[2, 3], shuffle=False))
    assert a == [[0, 1, 2, 3], [10, 11, 12, 13]]
    assert b == [[4, 5, 6, 7, 8, 9], [14, 15, 16, 17, 18, 19]]
    with pytest.raises(IndexError):
        S(range(20), pipeline_index=2, microbatch_size=2, num_microbatches=[2, 3])


def _train_worker(rank, world, tp=1):
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousParallelPlugin

    cfg = DecoderConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    ref = DecoderForCausalLM(cfg)
    torch.manual_seed(0)
    model = DecoderForCausalLM(cfg)
    ids = torch.randint(0, 128, (6, 32), generator=torch.Generator().manual_seed(3))
    # single process: mean over the 6 samples (3 micro-batches of 2)
    ref_opt = FusedAdamW(split_decay_groups(ref, 0.0), lr=1e-2)
    ref_loss = 0.0
    for i in range(3):
        sub = ids[2 * i : 2 * i + 2]
        l = ref(input_ids=sub, labels=sub).loss / 3
        l.backward()
        ref_loss += l.item()
    ref_grads = {n: p.grad.clone() for n, p in ref.named_parameters()}

    plugin = HeterogeneousParallelPlugin(tp_size=tp, microbatch_size=2, device=torch.device("cpu"))
    one = PipelineTemplate.even_split(model, 1)
    two = PipelineTemplate.even_split(model, 2)
    plugin.set_pipelines([one, two], {one: 1, two: 2})
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, crit, *_ = booster.boost(model, opt, criterion=lambda out, b: out.loss)
    pi = plugin._pipeline_index
    mine = ids[:2] if pi == 0 else ids[2:]
    out = booster.execute_pipeline(iter([{"input_ids": mine, "labels": mine}]), pmodel, crit, popt, return_loss=True)
    # weighted partial losses add up to the global mean
    part = out["loss"].clone() if out["loss"] is not None else torch.zeros(())
    dist.all_reduce(part)
    assert abs(part.item() / tp - ref_loss) < 1e-5, (part.item(), ref_loss)  # every tensor-parallel rank of a last stage reports the loss
    checked = 0
    for n, p in pmodel.module.named_parameters():
        if p.shape != ref_grads[n].shape:
            continue  # tensor-parallel shard: covered by the replicated parameters around it and by the loss
        assert torch.allclose(p.grad, ref_grads[n], atol=1e-5), (rank, n, (p.grad - ref_grads[n]).abs().max())
        checked += 1
    assert checked > 0 and plugin.train_batch_size == 6


def test_two_heterogeneous_pipelines_match_single_process():
    run_distributed(_train_worker, 3)


def test_two_heterogeneous_pipelines_with_tensor_parallelism():
    run_distributed(_train_worker, 6, 2)


def _replan_worker(rank, world, tmp):
    """Train a step with pipelines (1 stage | 2 stages), save, re-plan to (2 stages | 1 stage) on the same ranks with
    ``forced=True``, load the checkpoint: every rank then holds the trained weights of its NEW units, and the next step
    matches the single-process model."""
    import os

    from cornstarch_b200.booster import Booster
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousParallelPlugin

    cfg = DecoderConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=64)
    torch.manual_seed(0)
    ref = DecoderForCausalLM(cfg)
    torch.manual_seed(0)
    model = DecoderForCausalLM(cfg)
    ids = torch.randint(0, 128, (6, 32), generator=torch.Generator().manual_seed(3))

    def ref_step(opt):
        total = 0.0
        for i in range(3):
            sub = ids[2 * i : 2 * i + 2]
            l = ref(input_ids=sub, labels=sub).loss / 3
            l.backward()
            total += l.item()
        opt.step()
        opt.zero_grad()
        return total

    ref_opt = FusedAdamW(split_decay_groups(ref, 0.0), lr=1e-2)
    ref_step(ref_opt)

    plugin = HeterogeneousParallelPlugin(tp_size=1, microbatch_size=2, device=torch.device("cpu"))
    one, two = PipelineTemplate.even_split(model, 1), PipelineTemplate.even_split(model, 2)
    plugin.set_pipelines([one, two], {one: 1, two: 2})
    booster = Booster(plugin=plugin)
    pmodel, popt, crit, *_ = booster.boost(model, FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2), criterion=lambda out, b: out.loss)

    def my_batch():
        mine = ids[:2] if plugin._pipeline_index == 0 else ids[2:]
        if len(plugin.pipelines[plugin._pipeline_index].modules_per_stage) == 2 and plugin._pipeline_index == 0:
            mine = ids[:4]  # after the re-plan pipeline 0 is the deep one with two micro-batches
        elif plugin._pipeline_index == 1 and len(plugin.pipelines[1].modules_per_stage) == 1:
            mine = ids[4:]
        return {"input_ids": mine, "labels": mine}

    booster.execute_pipeline(iter([my_batch()]), pmodel, crit, popt, return_loss=True)
    popt.step()
    popt.zero_grad()
    ckpt = os.path.join(tmp, "model")
    booster.save_model(pmodel, ckpt, shard=True)
    booster.save_optimizer(popt, os.path.join(tmp, "optim"), shard=True)
    dist.barrier()

    # membership "changed": the deep pipeline now comes first
    plugin.set_pipelines([two, one], {two: 2, one: 1})
    pmodel, popt, crit, *_ = booster.boost(pmodel, popt, criterion=crit, forced=True)
    booster.load_model(pmodel, ckpt)
    booster.load_optimizer(popt, os.path.join(tmp, "optim"))  # Adam moments of the units this rank holds NOW, by name
    ref_sd = ref.state_dict()
    held = 0
    for n, p in pmodel.module.named_parameters():
        assert p.device.type == "cpu" and torch.allclose(p, ref_sd[n], atol=1e-5), (rank, n)
        held += 1
    assert held > 0
    out = booster.execute_pipeline(iter([my_batch()]), pmodel, crit, popt, return_loss=True)
    part = out["loss"].clone() if out["loss"] is not None else torch.zeros(())
    dist.all_reduce(part)
    want = ref_step(ref_opt)
    assert abs(part.item() - want) < 1e-4, (part.item(), want)
    # with the restored moments the second update lands on the single-process weights as well
    popt.step()
    ref_sd = ref.state_dict()
    for n, p in pmodel.module.named_parameters():
        assert torch.allclose(p, ref_sd[n], atol=2e-4), (rank, n, (p - ref_sd[n]).abs().max())  # 2 % of one update (lr 1e-2)


def test_replan_restores_released_units_and_continues(tmp_path):
    run_distributed(_replan_worker, 3, str(tmp_path))
