"""Plain data parallelism: every GPU holds the whole model; gradients live in a flat peer-mapped arena and are
averaged by one kernel launch per buffer (NCCL when the peer-memory path does not apply).  The counterpart of the
reference's examples/distributed/run_vlm_ddp.py, without ``DistributedDataParallel``'s per-bucket hooks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/distributed/run_vlm_ddp.py
    ... run_vlm_ddp.py --backend gloo --shape tiny      # on CPU
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import torch
import torch.distributed as dist

from cornstarch_b200.bench_support import SingleDeviceTrainer


def main():
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="vlm_small")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--backend", default="nccl", help="gloo runs the same script on CPU (use --shape tiny)")
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        device, kw = torch.device("cuda", torch.cuda.current_device()), {}
    else:
        device, kw = torch.device("cpu"), {"dtype": torch.float32}
    dist.init_process_group(a.backend)
    trainer = SingleDeviceTrainer(a.shape, samples_per_step=2, microbatch=1, device=device, dp_group=dist.group.WORLD, **kw)
    for step in range(a.steps):
        loss = trainer.step_e2e()
        if dist.get_rank() == 0:
            print(f"step {step} loss {float(loss):.4f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
