"""Modality-parallel hybrid training through the plugin API (the canonical script of the reference,
examples/distributed/run_vlm_hybrid.py): one pipeline template per modality, tensor parallelism inside every stage,
``Booster.execute_pipeline`` in the loop.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/distributed/run_vlm_hybrid.py --shape vlm --tp 2 --llm-stages 3

Works with gloo on CPU for the tiny shape: ``--shape tiny --tp 1 --llm-stages 1 --backend gloo`` on 2 processes.
A MoE language model with its experts sharded over the data-parallel replicas: ``--shape moe_tiny --ep 2 --backend gloo``
on 4 processes (2 replicas of encoder stage + LLM stage); ``--ep-capacity 1.25`` switches to the static-shape dispatch.
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import argparse

import torch
import torch.distributed as dist

from cornstarch_b200.booster import Booster
from cornstarch_b200.optim.fused_adamw import FusedAdamW
from cornstarch_b200.pipeline_template import PipelineTemplate
from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin
from cornstarch_b200.zoo import build_model, synthetic_batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="tiny")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--llm-stages", type=int, default=1)
    ap.add_argument("--microbatches", type=int, default=4)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--ep", type=int, default=1, help="expert-parallel degree (= number of data-parallel replicas)")
    ap.add_argument("--ep-capacity", type=float, default=None, help="capacity factor of the static-shape expert dispatch")
    ap.add_argument("--backend", default="nccl")
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(a.backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if a.backend == "nccl" else torch.device("cpu")
    dtype = torch.bfloat16 if a.backend == "nccl" else torch.float32

    model = build_model(a.shape, device="meta", dtype=dtype)
    model.gradient_checkpointing_enable()
    vision = ModalParallelPlugin(tp_size=a.tp, pipeline_template=PipelineTemplate.even_split(model.vision_encoder, 1))
    llm = ModalParallelPlugin(tp_size=a.tp, pipeline_template=PipelineTemplate.even_split(model.language_model, a.llm_stages),
                              ep_size=a.ep, ep_capacity_factor=a.ep_capacity)
    plugin = MultimodalParallelPlugin(encoder_plugins={"vision": vision}, language_model_plugin=llm,
                                      precision="bf16" if a.backend == "nccl" else None,
                                      num_microbatches=a.microbatches, microbatch_size=1, max_norm=1.0, device=dev)
    booster = Booster(plugin=plugin)
    model, optimizer, criterion, *_ = booster.boost(model, FusedAdamW, criterion=lambda out, batch: out.loss)
    model.train()
    replica = plugin.pg_mesh.coords[0][plugin.pg_mesh.dp_axis]  # every data-parallel replica reads its own samples
    for step in range(a.steps):
        batch = synthetic_batch(a.shape, a.microbatches, seed=step * plugin.dp_size + replica, device=dev, dtype=dtype)
        out = booster.execute_pipeline(iter([batch]), model, criterion, optimizer, return_loss=True)
        optimizer.step()
        optimizer.zero_grad()
        if out["loss"] is not None:
            print(f"step {step} loss {float(out['loss']):.4f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
