"""Single-GPU VLM training: vision encoder + MLP projector + LLM in a plain loop (synthetic data, random init).

    python examples/pretrain_vlm.py --shape tiny --steps 5            # CPU works for the tiny shape
    python examples/pretrain_vlm.py --shape vlm_small --steps 5       # on a B200

Mirrors the flow of the reference's examples/pretrain_vlm.py: build the model, enable gradient checkpointing,
freeze what should not train, loop.
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))  # run from a source checkout

import argparse

import torch

from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
from cornstarch_b200.utils.metrics import StepLogger
from cornstarch_b200.zoo import SHAPES, build_model, synthetic_batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="tiny", choices=sorted(SHAPES))
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--freeze-encoder", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = build_model(a.shape, device=dev, dtype=dtype)
    model.gradient_checkpointing_enable()
    # (encoder, projector) trainability per modality; llm_mode=None keeps the LLM as it is (trainable)
    model.train(encoders_mode={"vision": (not a.freeze_encoder, True)}, llm_mode=True)
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-4, max_norm=1.0)
    log = StepLogger(tokens_per_step=a.batch * SHAPES[a.shape].seq_len)
    for step in range(a.steps):
        batch = synthetic_batch(a.shape, a.batch, seed=step, device=dev, dtype=dtype)
        log.begin()
        loss = model(**batch).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        log.end(loss=loss.item())


if __name__ == "__main__":
    main()
