"""Synthetic datasets and the shared training loop of the heterogeneous-pipeline examples."""

import argparse
import os

import torch
import torch.distributed as dist
from torch.utils.data import Dataset


class Tokens(Dataset):
    """Random token sequences; labels equal the inputs (the models shift them)."""

    def __init__(self, n=64, seq=64, vocab=1000):
        self.data = torch.randint(0, vocab, (n, seq), generator=torch.Generator().manual_seed(0))

    def __len__(self):
        return len(self.data)

    def __getitem__(self, i):
        return {"input_ids": self.data[i], "labels": self.data[i]}


class Images(Dataset):
    """Random images with a regression target of the pooled feature's width."""

    def __init__(self, n=64, size=32, width=128):
        g = torch.Generator().manual_seed(0)
        self.pixels = torch.randn(n, 3, size, size, generator=g)
        self.targets = torch.randn(n, width, generator=g)

    def __len__(self):
        return len(self.pixels)

    def __getitem__(self, i):
        return {"pixel_values": self.pixels[i], "targets": self.targets[i]}


def init_distributed():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nccl")
    ap.add_argument("--checkpoint", default=None, help="directory: save model and optimizer there after training and load them back")
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(a.backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if a.backend == "nccl" else torch.device("cpu")
    return a, dev


def train_heterogeneous(model, dataset, criterion, dev, checkpoint=None, steps=None):
    """Two data-parallel replicas of ``model``: a 1-stage pipeline with 3 micro-batches and a 2-stage pipeline with 5
    (micro-batch size 2, global batch 16).  Needs 3 processes."""
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousParallelPlugin

    plugin = HeterogeneousParallelPlugin(tp_size=1, microbatch_size=2, device=dev)
    one, two = PipelineTemplate.even_split(model, 1), PipelineTemplate.even_split(model, 2)
    plugin.set_pipelines([one, two], {one: 3, two: 5})
    booster = Booster(plugin=plugin)
    loader = plugin.prepare_dataloader(dataset, shuffle=False)
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-3)
    model, opt, criterion, loader, _ = booster.boost(model, opt, criterion=criterion, dataloader=loader)
    for step, batch in enumerate(loader):
        if steps is not None and step >= steps:
            break
        batch = {k: v.to(dev) for k, v in batch.items()}
        out = booster.execute_pipeline(iter([batch]), model, criterion, opt, return_loss=True)
        opt.step()
        opt.zero_grad()
        if out["loss"] is not None:
            print(f"rank {dist.get_rank()} step {step} weighted loss {float(out['loss']):.4f}", flush=True)
    if checkpoint is not None:
        booster.save_model(model, os.path.join(checkpoint, "model"), shard=True)
        booster.save_optimizer(opt, os.path.join(checkpoint, "optimizer"), shard=True)
        dist.barrier()
        booster.load_model(model, os.path.join(checkpoint, "model"))
        booster.load_optimizer(opt, os.path.join(checkpoint, "optimizer"))
        if dist.get_rank() == 0:
            print("checkpoint written and read back:", sorted(os.listdir(checkpoint)), flush=True)
    return model, opt
