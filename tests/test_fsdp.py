"""FSDP2 around a tiny vision-language model (2 gloo ranks): same loss and same updated weights as the unsharded model
trained on the two ranks' batches with averaged gradients."""

import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _worker(rank, world):
    from cornstarch_b200 import zoo
    from cornstarch_b200.parallel.fsdp import shard_fully

    torch.manual_seed(0)
    ref = zoo.build_model("tiny", device="cpu", dtype=torch.float32)
    torch.manual_seed(0)
    model = zoo.build_model("tiny", device="cpu", dtype=torch.float32)
    model.gradient_checkpointing_enable()  # layers and projector recompute their forward while parameters are sharded
    model.train()
    shard_fully(model)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.1)

    batches = [zoo.synthetic_batch("tiny", 2, seed=r) for r in range(world)]
    loss = model(**batches[rank]).loss
    loss.backward()
    opt.step()

    ref_losses = [ref(**b).loss for b in batches]
    (sum(ref_losses) / world).backward()
    ref_opt.step()
    assert torch.allclose(loss.detach(), ref_losses[rank].detach(), atol=1e-5)

    full = {k: (v.full_tensor() if hasattr(v, "full_tensor") else v) for k, v in model.state_dict().items()}
    for k, v in ref.state_dict().items():
        assert torch.allclose(full[k], v, atol=1e-5), (k, (full[k] - v).abs().max())


def test_fsdp2_matches_unsharded():
    run_distributed(_worker, 2)
