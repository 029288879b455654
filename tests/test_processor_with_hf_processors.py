"""``MultimodalProcessor`` with real Hugging Face processors (built from their default constructors, nothing downloaded):
the default feature-count functions are picked by processor class and the placeholder tokens are expanded accordingly."""

import numpy as np
import pytest
import torch

tf = pytest.importorskip("transformers")


def _tokenizer(vocab):
    import sys
    import os

    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples"))
    from commons import WhitespaceTokenizer

    return WhitespaceTokenizer(vocab)


def test_image_and_audio_processors_from_transformers():
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
    from cornstarch_b200.models.vision import SiglipVisionConfig, SiglipVisionModel
    from cornstarch_b200.models.whisper import WhisperConfig, WhisperEncoder
    from cornstarch_b200.multimodal import ModalEncoderModule, MultimodalModel, MultimodalProcessor

    torch.manual_seed(0)
    llm = DecoderForCausalLM(DecoderConfig(vocab_size=512, hidden_size=32, intermediate_size=64, num_hidden_layers=1,
                                           num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256))
    vis = SiglipVisionModel(SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                               image_size=28, patch_size=14))
    aud = WhisperEncoder(WhisperConfig(num_mel_bins=16, d_model=32, encoder_layers=1, encoder_attention_heads=4, encoder_ffn_dim=64,
                                       max_source_positions=50))
    model = MultimodalModel(encoders={"vision": ModalEncoderModule(vis), "audio": ModalEncoderModule(aud)}, language_model=llm,
                            init_projector_type="mlp")
    image_proc = tf.SiglipImageProcessor(size={"height": 28, "width": 28})
    audio_proc = tf.WhisperFeatureExtractor(feature_size=16, chunk_length=1, sampling_rate=16000, hop_length=160)  # 100 frames -> 50 positions
    proc = MultimodalProcessor({"vision": image_proc, "audio": audio_proc}, _tokenizer(512), model,
                               predefined_tokens={"vision": "<image>", "audio": "<audio>"})
    images = [np.random.randint(0, 255, (40, 60, 3), dtype=np.uint8) for _ in range(2)]
    waves = [np.random.randn(16000).astype(np.float32) for _ in range(2)]
    batch = proc(encoder_inputs={"vision": {"images": images}, "audio": {"raw_speech": waves, "sampling_rate": 16000}},
                 llm_inputs={"text": ["<image> look <audio> listen", "<audio> first then <image>"]})
    assert list(batch.keys())[0] == "input_ids"
    ids = batch["input_ids"]
    assert (ids == model.token_ids["vision"]).sum(dim=1).tolist() == [4, 4]      # (28 / 14)^2 patches
    assert (ids == model.token_ids["audio"]).sum(dim=1).tolist() == [50, 50]     # max_source_positions
    assert tuple(batch["pixel_values"].shape) == (2, 3, 28, 28) and tuple(batch["input_features"].shape) == (2, 16, 100)
    out = model(input_ids=ids, pixel_values=batch["pixel_values"].float(), input_features=batch["input_features"].float(), labels=ids)
    assert torch.isfinite(out.loss)


def test_hugging_face_fast_tokenizer():
    """A ``PreTrainedTokenizerFast`` (word-level, built in memory): the modality token becomes an added special token and its
    id goes to the model.  The id may lie beyond the embedding table: placeholder positions are filled with encoder features
    and never looked up (nor used as labels), as in the reference."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    from cornstarch_b200 import zoo
    from cornstarch_b200.multimodal import MultimodalProcessor

    words = ["<pad>", "<unk>", "look", "listen"] + [f"w{i}" for i in range(996)]  # exactly the model's 1000 embeddings
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    hf_tok = tf.PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", unk_token="<unk>")
    model = zoo.build_model("tiny", dtype=torch.float32)

    class Images:
        def __call__(self, images=None, return_tensors="pt"):
            return {"pixel_values": torch.stack(images)}

    proc = MultimodalProcessor({"vision": Images()}, hf_tok, model, predefined_tokens={"vision": "<image>"},
                               num_feature_calculation_funcs={"vision": lambda i, o: [16] * len(o["pixel_values"])})
    assert model.token_ids == {"vision": 1000} and len(hf_tok) == 1001
    assert model.language_model.get_input_embeddings().weight.shape[0] == 1000
    batch = proc(encoder_inputs={"vision": {"images": [torch.randn(3, 56, 56)] * 2}},
                 llm_inputs={"text": ["<image> look w1 w2", "listen <image>"], "padding": True})
    assert (batch["input_ids"] == 1000).sum(dim=1).tolist() == [16, 16]
    out = model(input_ids=batch["input_ids"], pixel_values=batch["pixel_values"], labels=batch["input_ids"])
    assert torch.isfinite(out.loss)
