"""Trainer objects used by ``bench.py``: the same public calls a user script makes, packaged per parallel plan.

* 1 GPU: ``MultimodalModel`` + ``FusedAdamW`` in a plain loop with gradient accumulation.
* N GPUs: ``Booster(plugin=MultimodalParallelPlugin(...))`` and ``booster.execute_pipeline`` (modality-parallel
  pipeline with tensor parallelism), or plain data parallelism when asked for.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .optim.fused_adamw import FusedAdamW, split_decay_groups
from .zoo import SHAPES, build_model, synthetic_batch


class SingleDeviceTrainer:
    parallelism = "single"

    def __init__(self, shape: str, samples_per_step: int, microbatch: int, device, lr: float = 1e-4, seed: int = 0,
                 dp_group=None):
        self.shape = SHAPES[shape]
        self.model_name = _model_name(shape)
        self.seq_len = self.shape.seq_len
        self.samples = samples_per_step
        self.microbatch = microbatch
        self.device = device
        self.dp_group = dp_group
        self.world = dist.get_world_size(dp_group) if dp_group is not None else 1
        torch.manual_seed(seed)
        self.model = build_model(shape, device=device, dtype=torch.bfloat16)
        self.model.gradient_checkpointing_enable()
        self.model.train()
        self.opt = FusedAdamW(split_decay_groups(self.model, 0.01), lr=lr, max_norm=1.0)
        self.n_micro = samples_per_step // microbatch
        rank = dist.get_rank(dp_group) if dp_group is not None else 0
        self.host = [synthetic_batch(shape, microbatch, seed=1000 * rank + i, dtype=torch.bfloat16, pin=True)
                     for i in range(self.n_micro)]
        self.dev = [{k: v.to(device) for k, v in b.items()} for b in self.host]
        self.global_batch = samples_per_step * self.world
        self.tokens_per_step = self.global_batch * self.seq_len
        self.h2d_bytes_per_step = sum(v.numel() * v.element_size() for b in self.host for v in b.values())
        self.d2h_bytes_per_step = 4
        if self.world > 1:
            self.parallelism = f"dp{self.world}"

    def _run(self, batches):
        total = None
        for b in batches:
            out = self.model(**b)
            loss = out.loss / self.n_micro
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.world > 1:
            for g in self.opt.flat_grads():
                dist.all_reduce(g, op=dist.ReduceOp.AVG, group=self.dp_group)
        self.opt.step()
        self.opt.zero_grad()
        return total

    def step_device(self):
        return self._run(self.dev)

    def step_e2e(self) -> float:
        batches = [{k: v.to(self.device, non_blocking=True) for k, v in b.items()} for b in self.host]
        return float(self._run(batches).item())


def _model_name(shape: str) -> str:
    return {
        "vlm": "SigLIP-so400m-shape (27L,h1152) + MLP projector + Llama-3.1-8B-shape (32L,h4096,vocab 128256)",
        "valm": "SigLIP-so400m-shape + Whisper-large-v3-shape + Llama-3.1-8B-shape",
        "moe": "SigLIP-so400m-shape + Mixtral-8x7B-shape",
    }.get(shape, shape)


def build_trainer(args, rank: int, world: int, local_rank: int):
    device = torch.device("cuda", local_rank)
    plan = args.parallelism
    if world == 1:
        return SingleDeviceTrainer(args.shape, args.samples_per_gpu, args.microbatch, device)
    if plan == "dp":
        return SingleDeviceTrainer(args.shape, args.samples_per_gpu, args.microbatch, device, dp_group=dist.group.WORLD)
    from .bench_parallel import PipelineTrainer

    return PipelineTrainer(args, rank, world, device)
