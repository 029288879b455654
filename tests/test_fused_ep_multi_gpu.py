"""Expert-parallel MoE block on 2 GPUs: token dispatch / combine through the peer-memory push kernel against the NCCL
all-to-all path (outputs, input gradients, router and expert gradients), several calls in a row."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from cornstarch_b200.models.moe import MixtralConfig, MixtralSparseMoeBlock
        from cornstarch_b200.ops import _native as nat
        from cornstarch_b200.parallel import ep as EP

        cfg = MixtralConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                            num_key_value_heads=2, num_local_experts=max(4, world), num_experts_per_tok=2)
        torch.manual_seed(0)
        blocks = []
        for _ in range(2):
            torch.manual_seed(0)
            b = MixtralSparseMoeBlock(cfg).cuda().bfloat16()
            EP.shard_experts(b, dist.group.WORLD)
            blocks.append(b)
        for it in range(4):
            g = torch.Generator().manual_seed(100 * it + rank)
            x = torch.randn(2, 300 + 40 * it, 256, generator=g).cuda().bfloat16()
            res = []
            for fused, blk in zip((False, True), blocks):
                EP.FUSED_EP_ENABLED = fused
                blk.zero_grad()
                xi = x.clone().requires_grad_()
                y, _ = blk(xi)
                y.float().square().sum().backward()
                torch.cuda.synchronize()
                res.append((y.detach().float(), xi.grad.float(), blk.gate.weight.grad.float(), blk.experts[0].w1.weight.grad.float()))
            for name, a, b in zip(("y", "dx", "dgate", "dw1"), res[1], res[0]):
                err = (a - b).abs().max().item()
                assert err <= 2e-2 * max(1.0, b.abs().max().item()), (it, name, err)
        nat.check_status()
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback

        q.put((rank, traceback.format_exc()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_expert_exchange_two_gpus():
    from tests.dist_utils import free_port

    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    results = []
    while not q.empty():
        results.append(q.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert len(results) == 2 and all(r[1] == "ok" for r in results), results
