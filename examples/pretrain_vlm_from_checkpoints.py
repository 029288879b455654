"""Build a vision-language model from Hugging Face checkpoint DIRECTORIES (a vision encoder and an LLM; no network access
is needed or used) and train the new projector on synthetic data - the workflow of the reference's examples/pretrain_vlm.py
(``AutoModel.from_pretrained`` for both parts, projector created by ``MultimodalModel``, encoder and LLM frozen).

    python examples/pretrain_vlm_from_checkpoints.py --vision /path/to/siglip-or-clip-or-vit --llm /path/to/llama-like

Either directory may be that of a larger model: the vision tower is taken out of a two-tower CLIP / SigLIP checkpoint, the
decoder out of a vision-language checkpoint.  Without arguments the script first writes two tiny random checkpoints and
then loads them, so it runs anywhere.
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))  # run from a source checkout

import argparse
import tempfile

import torch

from cornstarch_b200.models import AutoModel
from cornstarch_b200.multimodal import ModalEncoderModule, MultimodalModel
from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups


def _tiny_checkpoints(root: str) -> tuple[str, str]:
    from cornstarch_b200.models.llama import LlamaConfig, LlamaForCausalLM
    from cornstarch_b200.models.vision import SiglipVisionConfig, SiglipVisionModel

    torch.manual_seed(0)
    SiglipVisionModel(SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                                         image_size=56, patch_size=14)).save_pretrained(os.path.join(root, "vision"))
    LlamaForCausalLM(LlamaConfig(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                 num_key_value_heads=2, max_position_embeddings=512)).save_pretrained(os.path.join(root, "llm"))
    return os.path.join(root, "vision"), os.path.join(root, "llm")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--vision", default=None, help="directory of a vision encoder checkpoint (config.json + weights)")
    ap.add_argument("--llm", default=None, help="directory of a causal LM checkpoint")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--text-tokens", type=int, default=64)
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev, dtype = (torch.device("cuda"), torch.bfloat16) if cuda else (torch.device("cpu"), torch.float32)
    if a.vision is None or a.llm is None:
        a.vision, a.llm = _tiny_checkpoints(tempfile.mkdtemp())

    vision = AutoModel.from_pretrained(a.vision, dtype=dtype, device=dev)
    llm = AutoModel.from_pretrained(a.llm, dtype=dtype, device=dev)
    model = MultimodalModel(encoders={"vision": ModalEncoderModule(vision)}, language_model=llm,
                            init_projector_type="mlp", init_activation="gelu").to(device=dev, dtype=dtype)
    image_token = llm.config.vocab_size - 1  # a real run registers "<image>" through MultimodalProcessor instead
    model.set_modality_token_ids({"vision": image_token})
    model.gradient_checkpointing_enable()
    model.train(encoders_mode={"vision": (False, True)}, llm_mode=False)  # only the projector trains
    trainable = [n for n, p in model.named_parameters() if p.requires_grad]
    print(f"{len(trainable)} trainable tensors, e.g. {trainable[:2]}", flush=True)

    vc = vision.config
    n_img = (vc.image_size // vc.patch_size) ** 2 + (1 if vc.model_type == "clip_vision_model" else 0)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-3, max_norm=1.0)
    g = torch.Generator().manual_seed(0)
    for step in range(a.steps):
        ids = torch.randint(0, image_token, (2, n_img + a.text_tokens), generator=g)
        ids[:, :n_img] = image_token
        pixels = torch.randn(2, 3, vc.image_size, vc.image_size, generator=g)
        loss = model(input_ids=ids.to(dev), pixel_values=pixels.to(dev, dtype), labels=ids.to(dev)).loss
        loss.backward()
        opt.step()
        opt.zero_grad()
        print(f"step {step} loss {loss.item():.4f}", flush=True)


if __name__ == "__main__":
    main()
