"""MultimodalModel behaviour on CPU: merging encoder outputs into the text, the bitfield mask rule, freezing by
``train(...)``, skipped modalities, projector save/load, the processor's token expansion, the timer aid and the
import-path aliases of the reference."""

import importlib

import pytest
import torch

from cornstarch_b200.zoo import build_model, synthetic_batch


def test_merge_places_features_and_builds_bitfield_mask():
    model = build_model("tiny", dtype=torch.float32)
    tid = model.token_ids["vision"]
    ids = torch.randint(0, 900, (2, 40))
    ids[:, 3:19] = tid
    feats = torch.randn(2, 16, model.language_model.config.hidden_size)
    embeds, bits = model.merge_encoder_outputs({"vision": (feats,)}, ids)
    assert torch.allclose(embeds[:, 3:19], feats)
    want_text = model.language_model.get_input_embeddings()(ids[:, :3])
    assert torch.allclose(embeds[:, :3], want_text)
    text_bits = (1 << 62) | 1 | 2
    assert bits[0, 0].item() == text_bits and bits[0, 5].item() == 2  # text sees every modality; the image has bit 1
    with pytest.raises(ValueError):
        model.check_counts = True
        model.merge_encoder_outputs({"vision": (feats[:, :5],)}, ids)


def test_labels_at_modality_positions_are_ignored_and_missing_modality_is_skipped():
    model = build_model("tiny", dtype=torch.float32)
    batch = synthetic_batch("tiny", 2, seed=1)
    out = model(**batch)
    assert torch.isfinite(out.loss)
    # text-only batch: the encoder has no input and is skipped
    ids = torch.randint(0, 900, (2, 32))
    out2 = model(input_ids=ids, labels=ids)
    assert torch.isfinite(out2.loss)


def test_train_modes_toggle_requires_grad():
    model = build_model("tiny", dtype=torch.float32)
    model.train(encoders_mode={"vision": (False, True)}, llm_mode=False)
    enc = model.vision_encoder
    assert not any(p.requires_grad for p in enc.module.parameters())
    assert all(p.requires_grad for p in enc.projector.parameters())
    assert not any(p.requires_grad for p in model.language_model.parameters())
    model.train(encoders_mode=None, llm_mode=True)
    assert all(p.requires_grad for p in model.language_model.parameters())
    assert not any(p.requires_grad for p in enc.module.parameters())  # None leaves a part as it was


def test_projector_save_and_load(tmp_path):
    from cornstarch_b200.multimodal import MultimodalProjector

    model = build_model("tiny", dtype=torch.float32)
    proj = model.vision_encoder.projector
    proj.save_pretrained(str(tmp_path))
    assert (tmp_path / "config.json").exists() and (tmp_path / "model.safetensors").exists()
    again = MultimodalProjector.from_pretrained(str(tmp_path))
    assert set(again.state_dict()) == set(proj.state_dict()) == {"projection.in_proj.weight", "projection.in_proj.bias",
                                                                  "projection.out_proj.weight", "projection.out_proj.bias"}
    for k, v in proj.state_dict().items():
        assert torch.equal(v, again.state_dict()[k])


class _Tok:
    """Whitespace tokenizer with special tokens kept whole."""

    def __init__(self):
        self.vocab = {"<pad>": 0}

    def __len__(self):
        return 1000

    def add_special_tokens(self, d):
        for t in d["additional_special_tokens"]:
            self.vocab.setdefault(t, 990 + len(self.vocab))

    def convert_tokens_to_ids(self, t):
        return self.vocab[t]

    def __call__(self, text, return_tensors="pt", **kw):
        rows = []
        for s in text:
            for sp in list(self.vocab):
                s = s.replace(sp, f" {sp} ")
            rows.append([self.vocab.get(w, 1 + (hash(w) % 900)) for w in s.split()])
        n = max(len(r) for r in rows)
        ids = torch.tensor([r + [0] * (n - len(r)) for r in rows])
        return {"input_ids": ids, "attention_mask": (ids != 0).long()}


class _ImageProc:
    def __call__(self, images=None, return_tensors="pt"):
        return {"pixel_values": torch.stack(images)}


def test_processor_expands_modality_tokens():
    from cornstarch_b200.multimodal import MultimodalProcessor

    model = build_model("tiny", dtype=torch.float32)
    proc = MultimodalProcessor({"vision": _ImageProc()}, _Tok(), model, predefined_tokens={"vision": "<image>"},
                               num_feature_calculation_funcs={"vision": lambda inputs, outputs: [16] * len(outputs["pixel_values"])})
    imgs = [torch.randn(3, 56, 56), torch.randn(3, 56, 56)]
    batch = proc(encoder_inputs={"vision": {"images": imgs}}, llm_inputs={"text": ["<image> a b c", "x <image> y"]})
    assert list(batch.keys())[0] == "input_ids"
    tid = model.token_ids["vision"]
    assert (batch["input_ids"] == tid).sum(dim=1).tolist() == [16, 16]
    out = model(input_ids=batch["input_ids"], pixel_values=batch["pixel_values"], labels=batch["input_ids"])
    assert torch.isfinite(out.loss)


def test_timer_context_manager_restores_functions():
    from cornstarch_b200.testing.timer import TimerContextManager

    import torch.nn.functional as F

    orig = F.gelu
    with TimerContextManager("torch.nn.functional.gelu") as t:
        assert F.gelu is not orig
        F.gelu(torch.randn(8))
        F.gelu(torch.randn(8))
    assert F.gelu is orig
    times = t.get_elapsed_times()
    assert len(times["torch.nn.functional.gelu"]) == 2 and all(x >= 0 for x in times["torch.nn.functional.gelu"])


def test_reference_import_paths_resolve():
    import cornstarch_b200.compat  # noqa: F401

    m = importlib.import_module("cornstarch.models.multimodal_language_model")
    assert hasattr(m, "MultimodalModel") and hasattr(m, "ModalEncoderModule")
    p = importlib.import_module("cornstarch.plugin.multimodal_parallel_plugin")
    assert hasattr(p, "MultimodalParallelPlugin")
    for path, names in {
        "cornstarch.plugin.multimodal_parallel_plugin.multimodal_1f1b": ["MultimodalEncoderTrainingOneForwardOneBackwardSchedule", "MultimodalPipelineP2PCommunication"],
        "cornstarch.plugin.multimodal_parallel_plugin.modal_process_group_mesh": ["MultiModalProcessGroupMesh"],
        "cornstarch.plugin.multimodal_parallel_plugin.multimodal_parallel_checkpoint_io": ["MultimodalParallelCheckpointIO"],
        "cornstarch.plugin.encoders_colocated_plugin.encoders_colocated_plugin": ["EncodersColocatedMultimodalParallelPlugin"],
        "cornstarch.plugin.heterogeneous_parallel_plugin.heterogeneous_dataloader": ["HeterogeneousDataLoader"],
        "cornstarch.shardformer.policies.llama": ["LlamaForCausalLMPolicy", "LlamaModelPolicy"],
        "cornstarch.shardformer.policies.siglip": ["SiglipVisionModelPolicy"],
        "cornstarch.shardformer.layers.context_parallel_bitfield_attention": ["context_parallel_bitfield_attention_forward"],
        "cornstarch.shardformer.layers.utils": ["ContextParallelBatchSplitUtils"],
        "cornstarch.models.evaclip": ["EvaCLIPVisionModel", "EvaCLIPVisionConfig"],
        "cornstarch.models.intern_vit": ["InternVisionModel"],
        "cornstarch.kernel.bitfield_attention": ["bitfield_attn_func", "BitfieldUtils"],
        "cornstarch.testing.timer": ["TimerContextManager"],
        "colossalai.booster": ["Booster"],
    }.items():
        mod = importlib.import_module(path)
        assert all(hasattr(mod, n) for n in names), (path, [n for n in names if not hasattr(mod, n)])


def test_lora_adapters_train_only_low_rank_and_merge():
    from cornstarch_b200.lora import LoRALinear, add_lora, merge_lora
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM

    torch.manual_seed(0)
    cfg = DecoderConfig(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2)
    m = DecoderForCausalLM(cfg)
    ids = torch.randint(0, 100, (2, 16))
    base = m(input_ids=ids).logits.detach()
    wrapped = add_lora(m, r=4, alpha=8, target=("q_proj", "v_proj", "down_proj"))
    assert len(wrapped) == 6
    assert torch.allclose(m(input_ids=ids).logits, base, atol=1e-6)  # B starts at zero
    for mod in m.modules():
        if isinstance(mod, LoRALinear):
            torch.nn.init.normal_(mod.lora_B, std=0.05)
    changed = m(input_ids=ids, labels=ids)
    assert not torch.allclose(changed.logits if "logits" in changed else m(input_ids=ids).logits, base, atol=1e-4)
    changed.loss.backward()
    q = m.model.layers[0].self_attn.q_proj
    assert q.base.weight.grad is None and q.lora_A.grad is not None and q.lora_A.grad.abs().sum() > 0
    adapted = m(input_ids=ids).logits.detach()
    merge_lora(m)
    assert not any(isinstance(x, LoRALinear) for x in m.modules())
    assert torch.allclose(m(input_ids=ids).logits, adapted, atol=1e-4)


def test_recompute_keep_last_layers_same_gradients():
    """Keeping the activations of the last k decoder layers (no recomputation there) changes no gradient."""
    from cornstarch_b200 import zoo

    batch = zoo.synthetic_batch("tiny", 2, seed=3)
    grads = []
    for keep in (None, 0, 1, 99):
        torch.manual_seed(0)
        model = zoo.build_model("tiny", device="cpu", dtype=torch.float32)
        if keep is not None:
            model.gradient_checkpointing_enable({"keep_last_layers": keep})
        model.train()
        model(**batch).loss.backward()
        grads.append({n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    for g in grads[1:]:
        assert g.keys() == grads[0].keys()
        for n in g:
            assert torch.allclose(g[n], grads[0][n], atol=1e-6), n


def test_generate_is_greedy_over_the_merged_sequence():
    """Every generated token is the arg-max of the model's next-token logits for the prefix (image features merged in)."""
    from cornstarch_b200 import zoo

    torch.manual_seed(0)
    model = zoo.build_model("tiny", device="cpu", dtype=torch.float32).eval()
    batch = zoo.synthetic_batch("tiny", 2, seed=1)
    prompt = batch["input_ids"][:, :40]
    out = model.generate(prompt, max_new_tokens=3, pixel_values=batch["pixel_values"])
    assert out.shape == (2, 43) and torch.equal(out[:, :40], prompt)
    for t in range(40, 43):
        logits = model(input_ids=out[:, :t], pixel_values=batch["pixel_values"]).logits
        assert torch.equal(logits[:, -1].argmax(-1), out[:, t])
    # with an end-of-sequence id the finished rows keep emitting it
    eos = int(out[0, 40])
    out2 = model.generate(prompt, max_new_tokens=3, eos_token_id=eos, pixel_values=batch["pixel_values"])
    assert bool((out2[0, 40:] == eos).all())


def test_recompute_tuner_two_passes(monkeypatch):
    """Pass one keeps what the upper estimate allows; pass two re-measures what a kept layer cost and keeps more."""
    from cornstarch_b200 import zoo
    from cornstarch_b200.utils import recompute as R

    model = zoo.build_model("tiny", device="cpu", dtype=torch.float32)
    model.gradient_checkpointing_enable()
    n_layers = len(model.language_model.model.layers)
    est = R.activation_bytes_per_layer(model.language_model.config, 256, 1)
    mem = {"free": 6 * 2**30 + int(1.5 * est), "reserved": 10 * 2**30}
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda *a, **k: (mem["free"], 180 * 2**30))
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda *a, **k: mem["reserved"])
    tuner = R.RecomputeTuner(model, 256, 1, 1)
    assert tuner.after_step() == 1  # room for one estimated layer above the safety margin
    assert model.language_model.model.recompute_keep_layers == 1
    # the kept layer turned out to cost 0.6 of the estimate; the driver still reports room for one more such layer
    mem["reserved"] += int(0.6 * est)
    mem["free"] = 6 * 2**30 + int(0.7 * est)
    assert tuner.after_step() == min(n_layers, 2)
    assert tuner.after_step() == min(n_layers, 2)  # further calls change nothing
