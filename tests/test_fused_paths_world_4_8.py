"""The fused peer-memory paths beyond two ranks: the same workers as the two-GPU tests (fused GEMM + all-reduce,
gradient all-reduce / reduce-scatter kernel, context-parallel attention with K/V pulled from the peers, expert
dispatch / combine) on 4 and on 8 GPUs of one node.  Skipped where fewer GPUs are visible."""

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _run(worker, world, timeout=420):
    from tests.dist_utils import free_port

    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    results = []
    while not q.empty():
        results.append(q.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert len(results) == world and all(r[1] == "ok" for r in results), results


def _need(world):
    return pytest.mark.skipif(torch.cuda.device_count() < world, reason=f"needs {world} GPUs")


@pytest.mark.parametrize("world", [pytest.param(4, marks=_need(4)), pytest.param(8, marks=_need(8))])
def test_gemm_allreduce(world):
    from tests.test_fused_tp_multi_gpu import _worker

    _run(_worker, world)


@pytest.mark.parametrize("world", [pytest.param(4, marks=_need(4)), pytest.param(8, marks=_need(8))])
def test_gradient_reduce_kernel(world):
    from tests.test_fused_tp_multi_gpu import _grad_reduce_worker

    _run(_grad_reduce_worker, world)


@pytest.mark.parametrize("world", [pytest.param(4, marks=_need(4)), pytest.param(8, marks=_need(8))])
def test_context_parallel_attention(world):
    from tests.test_fused_cp_multi_gpu import _worker

    _run(_worker, world)


@pytest.mark.parametrize("world", [pytest.param(4, marks=_need(4)), pytest.param(8, marks=_need(8))])
def test_expert_exchange(world):
    from tests.test_fused_ep_multi_gpu import _worker

    _run(_worker, world)
