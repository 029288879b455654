"""LoRA fine-tuning of the LLM of a VLM: encoder frozen, projector trained, low-rank adapters on the attention
projections of the language model (the flow of the reference's examples/pretrain_vlm_lora.py, without ``peft``).

    python examples/pretrain_vlm_lora.py --shape tiny --steps 3
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))  # run from a source checkout

import argparse

import torch

from cornstarch_b200.lora import add_lora
from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
from cornstarch_b200.zoo import SHAPES, build_model, synthetic_batch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="tiny", choices=sorted(SHAPES))
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = build_model(a.shape, device=dev, dtype=dtype)
    model.train(encoders_mode={"vision": (False, True)}, llm_mode=False)   # freeze encoder and LLM, train the projector
    wrapped = add_lora(model.language_model, r=16, alpha=32, target=("q_proj", "k_proj", "v_proj", "o_proj"))
    print(f"{len(wrapped)} projections adapted;",
          sum(p.numel() for p in model.parameters() if p.requires_grad), "trainable parameters")
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-4)
    for step in range(a.steps):
        batch = synthetic_batch(a.shape, 2, seed=step, device=dev, dtype=dtype)
        loss = model(**batch).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        print(step, loss.item())


if __name__ == "__main__":
    main()
