"""The benchmark's expert-parallel and context-parallel trainers on CPU-sized shapes: loss of the first step equals
the single-process model on the same data, and a step updates the weights."""

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _ep_worker(rank, world):
    from cornstarch_b200.bench_support import ExpertParallelTrainer, SingleDeviceTrainer

    dev = torch.device("cpu")
    ref = SingleDeviceTrainer("moe_tiny", 2, 1, dev, dtype=torch.float32)
    ref.host = None
    tr = ExpertParallelTrainer("moe_tiny", 2, 1, dev, dist.group.WORLD, dtype=torch.float32)
    assert len(tr.model.language_model.model.layers[0].block_sparse_moe.experts) == 4 // world
    # loss on this rank's data against the unsharded model with the same seed
    from cornstarch_b200.zoo import build_model

    torch.manual_seed(0)
    full = build_model("moe_tiny", dtype=torch.float32)
    want = sum(full(**b).loss.item() for b in tr.dev) / tr.n_micro
    got = float(tr.step_device())
    assert abs(got - want) < 1e-4, (got, want)
    l2 = float(tr.step_device())
    assert l2 < got  # the step trained
    assert "ep" in tr.parallelism and tr.global_batch == 2 * world


def _cp_worker(rank, world):
    from cornstarch_b200.bench_support import ContextParallelTrainer
    from cornstarch_b200.zoo import build_model

    dev = torch.device("cpu")
    tr = ContextParallelTrainer("long_tiny", 2, 1, dev, dist.group.WORLD, dtype=torch.float32)
    torch.manual_seed(0)
    full = build_model("long_tiny", dtype=torch.float32, mask_mode="instance")
    want = sum(full(**b).loss.item() for b in tr.dev) / tr.n_micro
    # every rank reports sp * (its local token loss sum) / global count: the mean over ranks is the global loss
    got = tr.step_device().clone()
    dist.all_reduce(got)
    got = float(got) / world
    assert abs(got - want) < 1e-4, (got, want)
    assert tr.tokens_per_step == 2 * 1024


def test_expert_parallel_trainer():
    run_distributed(_ep_worker, 2)


def test_context_parallel_trainer():
    run_distributed(_cp_worker, 2)


def _pipeline_worker(rank, world):
    """The benchmark's modality-parallel pipeline trainer (encoder stage + LLM stage, tp 2) steps, tunes recomputation
    (a no-op without a GPU, but through the same group logic) and steps again."""
    from types import SimpleNamespace

    from cornstarch_b200.bench_parallel import PipelineTrainer

    args = SimpleNamespace(shape="tiny", parallelism="enc1+llm1xtp2", samples_per_gpu=1, microbatch=1)
    tr = PipelineTrainer(args, rank, world, torch.device("cpu"))
    l1 = tr.step_device()
    keep = tr.tune_recompute()
    assert keep == 0 and "decoder layers kept" in tr.recompute
    l2 = tr.step_device()
    if tr.is_last:
        assert torch.isfinite(l1) and torch.isfinite(l2)
    assert tr.global_batch == world
    # what bench.py asks of a trainer after the timed steps: replicated parameters agree inside the tensor-parallel pair
    assert "stage" in tr.role and "tp rank" in tr.role
    c = tr.checks()
    assert c["tp_replicated"]["ranks"] == 2 and c["tp_replicated"]["params"] > 0
    assert c["tp_replicated"]["mismatched"] == 0, c


def test_pipeline_trainer_with_recompute_tuning():
    run_distributed(_pipeline_worker, 4)


def _tp_worker(rank, world, seq_shard):
    """The benchmark's tensor-parallel trainer (language model over both ranks, encoder replicated) in both activation
    layouts: two steps, finite loss, replicated parameters still equal on both ranks."""
    import os

    os.environ["CORNSTARCH_B200_TP_SEQ_SHARD"] = "1" if seq_shard else "0"
    from cornstarch_b200.bench_support import TensorParallelTrainer

    tr = TensorParallelTrainer("tiny", 2, 1, torch.device("cpu"), dist.group.WORLD, dtype=torch.float32)
    l1 = tr.step_device()
    l2 = tr.step_device()
    assert torch.isfinite(l1) and torch.isfinite(l2)
    assert ("token-sharded" in tr.parallelism) == seq_shard
    c = tr.checks()
    assert c["tp_replicated"]["params"] > 0 and c["tp_replicated"]["mismatched"] == 0, c
    # both layouts compute the same function: the loss of the first step is the single-process loss
    everyone = [None, None]
    dist.all_gather_object(everyone, float(l1))
    assert abs(everyone[0] - everyone[1]) < 1e-5


@pytest.mark.parametrize("seq_shard", [False, True])
def test_tensor_parallel_trainer(seq_shard):
    run_distributed(_tp_worker, 2, seq_shard)
