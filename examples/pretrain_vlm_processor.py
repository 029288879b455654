"""Single-GPU (or CPU) VLM training through ``MultimodalProcessor``: images and text go through an image processor and a
tokenizer, the image token is expanded to one copy per encoder feature, and a ``DataLoader`` collates batches - the flow
of the reference's examples/pretrain_vlm.py:83-146, with offline stand-ins for the Hugging Face processors.

    python examples/pretrain_vlm_processor.py --steps 3
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))  # run from a source checkout
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import argparse
from functools import partial

import torch
from commons import ResizeImageProcessor, WhitespaceTokenizer, collate_fn
from fake_dataset import FakeVisionDataset
from torch.utils.data import DataLoader

from cornstarch_b200.multimodal import MultimodalProcessor
from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
from cornstarch_b200.zoo import SHAPES, build_model


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default=None)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=2)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev, dtype = (torch.device("cuda"), torch.bfloat16) if cuda else (torch.device("cpu"), torch.float32)
    shape = SHAPES[a.shape or ("vlm_small" if cuda else "tiny")]
    model = build_model(shape, device=dev, dtype=dtype)
    model.gradient_checkpointing_enable()
    model.train(encoders_mode={"vision": (False, True)}, llm_mode=True)  # frozen encoder, trainable projector and LLM

    processor = MultimodalProcessor(
        encoder_processors={"vision": ResizeImageProcessor(shape.image_size)},
        llm_tokenizer=WhitespaceTokenizer(shape.vocab), model=model, predefined_tokens={"vision": "<image>"},
        num_feature_calculation_funcs={"vision": lambda inputs, outputs: [shape.image_tokens] * len(outputs["pixel_values"])})
    words = max(8, shape.seq_len - shape.image_tokens - 8)
    loader = DataLoader(FakeVisionDataset(n=a.steps * a.batch, words=min(words, 256)), batch_size=a.batch,
                        collate_fn=partial(collate_fn, processor=processor, dtype=dtype))
    opt = FusedAdamW(split_decay_groups(model, 0.01), lr=1e-4, max_norm=1.0)
    for step, batch in enumerate(loader):
        batch = {k: v.to(dev) for k, v in batch.items()}
        loss = model(**batch).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        n_img = int((batch["input_ids"] == model.token_ids["vision"]).sum())
        print(f"step {step} loss {loss.item():.4f} ({n_img} image positions, {batch['input_ids'].numel()} tokens)", flush=True)


if __name__ == "__main__":
    main()
