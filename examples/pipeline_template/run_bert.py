"""Heterogeneous pipelines (Oobleck style): data-parallel replicas of one BERT are pipelines with different numbers of
stages and micro-batches (the reference's examples/pipeline_template/run_bert.py).  3 processes: one 1-stage pipeline
and one 2-stage pipeline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 3 --master-addr 127.0.0.1 \
        examples/pipeline_template/run_bert.py --backend gloo
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import argparse

import torch
import torch.distributed as dist
from torch.utils.data import Dataset

from cornstarch_b200.booster import Booster
from cornstarch_b200.models.text_legacy import BertConfig, BertForMaskedLM
from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
from cornstarch_b200.pipeline_template import PipelineTemplate
from cornstarch_b200.plugin.heterogeneous_parallel_plugin import HeterogeneousParallelPlugin


class Tokens(Dataset):
    def __init__(self, n=64, seq=64, vocab=1000):
        self.data = torch.randint(0, vocab, (n, seq), generator=torch.Generator().manual_seed(0))

    def __len__(self):
        return len(self.data)

    def __getitem__(self, i):
        return {"input_ids": self.data[i], "labels": self.data[i]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nccl")
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(a.backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if a.backend == "nccl" else torch.device("cpu")
    torch.manual_seed(0)
    model = BertForMaskedLM(BertConfig(num_hidden_layers=4, hidden_size=128, num_attention_heads=4, intermediate_size=256, vocab_size=1000, max_position_embeddings=64, tie_word_embeddings=False))
    plugin = HeterogeneousParallelPlugin(tp_size=1, microbatch_size=2, device=dev)
    one, two = PipelineTemplate.even_split(model, 1), PipelineTemplate.even_split(model, 2)
    plugin.set_pipelines([one, two], {one: 3, two: 5})  # 3 and 5 micro-batches of 2 samples: global batch 16
    booster = Booster(plugin=plugin)
    loader = plugin.prepare_dataloader(Tokens(), shuffle=False)
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-3)
    model, opt, criterion, loader, _ = booster.boost(model, opt, criterion=lambda out, batch: out.loss, dataloader=loader)
    for step, batch in enumerate(loader):
        batch = {k: v.to(dev) for k, v in batch.items()}
        out = booster.execute_pipeline(iter([batch]), model, criterion, opt, return_loss=True)
        opt.step()
        opt.zero_grad()
        if out["loss"] is not None:
            print(f"rank {dist.get_rank()} step {step} weighted loss {float(out['loss']):.4f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
