"""Plain data parallelism: every GPU holds the whole model; gradients live in a flat peer-mapped arena and are
averaged by one kernel launch per buffer (NCCL when the peer-memory path does not apply).  The counterpart of the
reference's examples/distributed/run_vlm_ddp.py, without ``DistributedDataParallel``'s per-bucket hooks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/run_vlm_ddp.py
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import torch
import torch.distributed as dist

from cornstarch_b200.bench_support import SingleDeviceTrainer


def main():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    trainer = SingleDeviceTrainer("vlm_small", samples_per_step=2, microbatch=1, device=torch.device("cuda", torch.cuda.current_device()),
                                  dp_group=dist.group.WORLD)
    for step in range(3):
        loss = trainer.step_e2e()
        if dist.get_rank() == 0:
            print(step, loss, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
