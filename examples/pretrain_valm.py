"""Vision + audio + language model on one GPU: SigLIP-shaped and Whisper-shaped encoders feed one LLM
(the flow of the reference's examples/pretrain_valm.py with synthetic pixels and log-mel features).

    python examples/pretrain_valm.py --steps 3
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))  # run from a source checkout

import argparse

import torch

from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
from cornstarch_b200.zoo import build_model, synthetic_batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda" if cuda else "cpu")
    shape, dtype = ("valm", torch.bfloat16) if cuda else ("valm_tiny", torch.float32)  # CPU: a toy shape of the same structure
    model = build_model(shape, device=dev, dtype=dtype)
    model.gradient_checkpointing_enable()
    model.train(encoders_mode={"vision": (False, True), "audio": (False, True)}, llm_mode=True)  # train projectors + LLM
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-4, max_norm=1.0)
    for step in range(a.steps):
        batch = synthetic_batch(shape, 1, seed=step, device=dev, dtype=dtype)
        loss = model(**batch).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        print(step, loss.item())


if __name__ == "__main__":
    main()
