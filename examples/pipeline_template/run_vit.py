"""Heterogeneous pipelines (Oobleck style) of a small ViT regressing a target from the pooled feature (the reference's
examples/pipeline_template/run_vit.py).  3 processes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 3 --master-addr 127.0.0.1 \
        examples/pipeline_template/run_vit.py --backend gloo
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist
from data_builder import Images, init_distributed, train_heterogeneous
from cornstarch_b200.models.vision import ViTConfig, ViTModel


def main():
    a, dev = init_distributed()
    torch.manual_seed(0)
    model = ViTModel(ViTConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=4,
                               image_size=32, patch_size=8))

    def criterion(out, batch):
        return (out.pooler_output.float() - batch["targets"].float()).square().mean()

    train_heterogeneous(model, Images(), criterion, dev, checkpoint=a.checkpoint)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
