"""Named model shapes and synthetic batches for the benchmark configurations.

``tiny``      2-layer ViT (hidden 64) + MLP projector + 2-layer Llama (hidden 128): CPU / gloo correctness runs.
``vlm``       SigLIP-so400m-shaped encoder + 2-layer GELU MLP projector + Llama-3.1-8B-shaped LLM, sequence 8192.
``valm``      ``vlm`` plus a Whisper-large-v3-shaped audio encoder (1500 audio tokens).
``moe``       SigLIP-so400m-shaped encoder + Mixtral-8x7B-shaped LLM, sequence 4096.
``vlm_small`` a 4-layer cut of ``vlm`` (same layer shapes) for smoke tests and profiler captures.
``long``      ``vlm`` at sequence 65536 with 8 images per sample at random positions (context parallelism).
``long_tiny`` / ``moe_tiny``  CPU-sized versions of ``long`` and ``moe`` for the gloo tests;
``long_small`` / ``moe_small``  4-layer cuts at the real layer shapes for multi-GPU smoke runs.

Weights are random-initialised; data is synthetic (pixels ~ N(0,1), token ids uniform), as there is no
network access for datasets or checkpoints.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .models.llama import DecoderConfig, DecoderForCausalLM
from .models.moe import MixtralConfig, MoeForCausalLM
from .models.vision import SiglipVisionConfig, SiglipVisionModel, ViTConfig, ViTModel
from .models.whisper import WhisperConfig, WhisperEncoder
from .multimodal.modeling import ModalEncoderModule, MultimodalModel, MultimodalProjector, MultimodalProjectorConfig


@dataclass
class Shape:
    name: str
    seq_len: int
    image_tokens: int = 0
    audio_tokens: int = 0
    image_size: int = 0
    mel_bins: int = 0
    mel_frames: int = 0
    vocab: int = 0
    llm: dict = field(default_factory=dict)
    vision: dict = field(default_factory=dict)
    audio: dict = field(default_factory=dict)
    moe: bool = False
    images_per_sample: int = 1


SIGLIP_SO400M = dict(hidden_size=1152, intermediate_size=4304, num_hidden_layers=27, num_attention_heads=16,
                     image_size=384, patch_size=14, hidden_act="gelu_pytorch_tanh", vision_use_head=False)
LLAMA31_8B = dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                  num_attention_heads=32, num_key_value_heads=8, rope_theta=500000.0, max_position_embeddings=8192,
                  rms_norm_eps=1e-5)
WHISPER_LARGE_V3 = dict(num_mel_bins=128, d_model=1280, encoder_layers=32, encoder_attention_heads=20,
                        encoder_ffn_dim=5120, max_source_positions=1500)
MIXTRAL_8X7B = dict(vocab_size=32000, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                    num_attention_heads=32, num_key_value_heads=8, num_local_experts=8, num_experts_per_tok=2,
                    rope_theta=1e6, max_position_embeddings=4096, rms_norm_eps=1e-5)

SHAPES = {
    "tiny": Shape("tiny", seq_len=256, image_tokens=16, image_size=56, vocab=1000,
                  llm=dict(vocab_size=1000, hidden_size=128, intermediate_size=352, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512),
                  vision=dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                              image_size=56, patch_size=14, hidden_act="gelu", vit=True)),
    "vlm": Shape("vlm", seq_len=8192, image_tokens=729, image_size=384, vocab=128256, llm=LLAMA31_8B, vision=SIGLIP_SO400M),
    "vlm_small": Shape("vlm_small", seq_len=8192, image_tokens=729, image_size=384, vocab=128256,
                       llm={**LLAMA31_8B, "num_hidden_layers": 4}, vision={**SIGLIP_SO400M, "num_hidden_layers": 3}),
    "valm": Shape("valm", seq_len=8192, image_tokens=729, audio_tokens=1500, image_size=384, mel_bins=128, mel_frames=3000,
                  vocab=128256, llm=LLAMA31_8B, vision=SIGLIP_SO400M, audio=WHISPER_LARGE_V3),
    "long": Shape("long", seq_len=65536, image_tokens=729, image_size=384, vocab=128256, images_per_sample=8,
                  llm={**LLAMA31_8B, "max_position_embeddings": 65536}, vision=SIGLIP_SO400M),
    "valm_tiny": Shape("valm_tiny", seq_len=256, image_tokens=16, audio_tokens=24, image_size=56, mel_bins=16, mel_frames=48, vocab=1000,
                       llm=dict(vocab_size=1000, hidden_size=128, intermediate_size=352, num_hidden_layers=2,
                                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512),
                       vision=dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   image_size=56, patch_size=14, hidden_act="gelu", vit=True),
                       audio=dict(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128,
                                  max_source_positions=24)),
    "long_small": Shape("long_small", seq_len=16384, image_tokens=729, image_size=384, vocab=128256, images_per_sample=8,
                        llm={**LLAMA31_8B, "num_hidden_layers": 4, "max_position_embeddings": 16384},
                        vision={**SIGLIP_SO400M, "num_hidden_layers": 3}),
    "moe_small": Shape("moe_small", seq_len=4096, image_tokens=729, image_size=384, vocab=32000, moe=True,
                       llm={**MIXTRAL_8X7B, "num_hidden_layers": 4}, vision={**SIGLIP_SO400M, "num_hidden_layers": 3}),
    "long_tiny": Shape("long_tiny", seq_len=1024, image_tokens=16, image_size=56, vocab=1000, images_per_sample=4,
                       llm=dict(vocab_size=1000, hidden_size=128, intermediate_size=352, num_hidden_layers=2,
                                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=1024),
                       vision=dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                   image_size=56, patch_size=14, hidden_act="gelu", vit=True)),
    "moe_tiny": Shape("moe_tiny", seq_len=256, image_tokens=16, image_size=56, vocab=1000, moe=True,
                      llm=dict(vocab_size=1000, hidden_size=128, intermediate_size=192, num_hidden_layers=2,
                               num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512,
                               num_local_experts=4, num_experts_per_tok=2),
                      vision=dict(hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                                  image_size=56, patch_size=14, hidden_act="gelu", vit=True)),
    "moe": Shape("moe", seq_len=4096, image_tokens=729, image_size=384, vocab=32000, llm=MIXTRAL_8X7B, vision=SIGLIP_SO400M,
                 moe=True),
}


def drop_cls_token(inputs, output):
    """ViT front-ends prepend a [CLS] token; the LLM only receives patch tokens."""
    h = output["last_hidden_state"] if isinstance(output, dict) else output[0]
    return (h[:, 1:],)


def build_model(shape: Shape | str, projector: str = "mlp", activation: str = "gelu_pytorch_tanh",
                device=None, dtype=None, mask_mode: str = "modality") -> MultimodalModel:
    """Instantiate the multimodal model of a named shape directly on ``device`` in ``dtype``."""
    sh = SHAPES[shape] if isinstance(shape, str) else shape
    ctx = torch.device(device) if device is not None else torch.device("cpu")
    prev = torch.get_default_dtype()
    if dtype is not None:
        torch.set_default_dtype(dtype)
    try:
        with ctx:
            llm_cfg = (MixtralConfig if sh.moe else DecoderConfig)(**sh.llm)
            llm = (MoeForCausalLM if sh.moe else DecoderForCausalLM)(llm_cfg)
            encoders = {}
            if sh.vision:
                v = dict(sh.vision)
                if v.pop("vit", False):
                    vcfg = ViTConfig(**v)
                    vis = ViTModel(vcfg, add_pooling_layer=False)
                    post = drop_cls_token
                else:
                    vcfg = SiglipVisionConfig(**v)
                    vis = SiglipVisionModel(vcfg)
                    post = None
                pcfg = MultimodalProjectorConfig(encoder_config=vcfg, text_config=llm_cfg, projection_type=projector,
                                                 activation=activation)
                kwargs = dict(postprocess_module_callback=post) if post else {}
                encoders["vision"] = ModalEncoderModule(vis, MultimodalProjector(pcfg), **kwargs)
            if sh.audio:
                acfg = WhisperConfig(**sh.audio)
                aud = WhisperEncoder(acfg)
                pcfg = MultimodalProjectorConfig(encoder_config=acfg, text_config=llm_cfg, projection_type=projector,
                                                 activation=activation)
                encoders["audio"] = ModalEncoderModule(aud, MultimodalProjector(pcfg))
            model = MultimodalModel(encoders=encoders, language_model=llm, mask_mode=mask_mode)
    finally:
        torch.set_default_dtype(prev)
    ids = {}
    if sh.vision:
        ids["vision"] = sh.vocab - 1
    if sh.audio:
        ids["audio"] = sh.vocab - 2
    model.set_modality_token_ids(ids)
    return model


def synthetic_batch(shape: Shape | str, batch: int, seed: int = 0, device="cpu", dtype=torch.float32, pin: bool = False):
    """One batch of the named shape: image (and audio) placeholders first, then text; labels = input ids."""
    sh = SHAPES[shape] if isinstance(shape, str) else shape
    g = torch.Generator().manual_seed(seed)
    n_special = (1 if sh.vision else 0) + (1 if sh.audio else 0)
    ids = torch.randint(0, sh.vocab - n_special, (batch, sh.seq_len), generator=g)
    pos = 0
    out = {}
    if sh.vision and sh.images_per_sample > 1:
        # one image somewhere inside each of `images_per_sample` equal segments of the sequence
        seg = sh.seq_len // sh.images_per_sample
        for b in range(batch):
            for i in range(sh.images_per_sample):
                start = i * seg + int(torch.randint(0, seg - sh.image_tokens, (1,), generator=g))
                ids[b, start : start + sh.image_tokens] = sh.vocab - 1
        out["pixel_values"] = torch.randn(batch * sh.images_per_sample, 3, sh.image_size, sh.image_size, generator=g).to(dtype)
    elif sh.vision:
        ids[:, pos : pos + sh.image_tokens] = sh.vocab - 1
        pos += sh.image_tokens
        out["pixel_values"] = torch.randn(batch, 3, sh.image_size, sh.image_size, generator=g).to(dtype)
    if sh.audio:
        ids[:, pos : pos + sh.audio_tokens] = sh.vocab - 2
        pos += sh.audio_tokens
        out["input_features"] = torch.randn(batch, sh.mel_bins, sh.mel_frames, generator=g).to(dtype)
    out["input_ids"] = ids
    out["labels"] = ids.clone()
    if pin and torch.cuda.is_available():
        out = {k: v.pin_memory() for k, v in out.items()}
    if torch.device(device).type != "cpu":
        out = {k: v.to(device, non_blocking=True) for k, v in out.items()}
    return out
