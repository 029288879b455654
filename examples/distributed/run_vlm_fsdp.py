"""Fully-sharded data parallelism (PyTorch FSDP2) around a vision-language model of this package: every transformer
layer of the encoder and of the language model is one sharding unit.  The counterpart of the reference's
examples/distributed/run_vlm_fsdp.py.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/run_vlm_fsdp.py
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import torch
import torch.distributed as dist

from cornstarch_b200 import zoo
from cornstarch_b200.parallel.fsdp import shard_fully


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl" if use_cuda else "gloo")
    device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if use_cuda else torch.float32
    shape = os.environ.get("SHAPE", "vlm_small" if use_cuda else "tiny")

    torch.manual_seed(0)  # the same initial weights on every rank; fully_shard keeps each rank's slice
    model = zoo.build_model(shape, device=device, dtype=dtype)
    model.gradient_checkpointing_enable()
    shard_fully(model)
    optimizer = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=use_cuda)

    for step in range(3):
        batch = zoo.synthetic_batch(shape, 1, seed=step * dist.get_world_size() + dist.get_rank(), device=device, dtype=dtype)
        loss = model(**batch).loss
        loss.backward()
        optimizer.step()
        optimizer.zero_grad()
        if dist.get_rank() == 0:
            print(step, float(loss.detach()), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
