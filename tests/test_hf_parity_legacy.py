"""GPT-2, BERT and OPT: state dicts load from the HF implementations unchanged and losses / logits agree (fp32, CPU)."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _load(ours, hf):
    missing, unexpected = ours.load_state_dict(hf.state_dict(), strict=False)
    assert not [m for m in missing if "rotary" not in m], missing
    assert not unexpected, unexpected


def test_gpt2_matches_hf():
    from transformers import GPT2Config as HC, GPT2LMHeadModel as HM

    from cornstarch_b200.models.text_legacy import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(0)
    hf = HM(HC(n_layer=2, n_embd=32, n_head=4, vocab_size=100, n_positions=64, resid_pdrop=0, embd_pdrop=0, attn_pdrop=0)).eval()
    ours = GPT2LMHeadModel(GPT2Config(n_layer=2, n_embd=32, n_head=4, vocab_size=100, n_positions=64)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (2, 24))
    want = hf(input_ids=ids, labels=ids)
    got = ours(input_ids=ids, labels=ids)
    assert torch.allclose(got.loss, want.loss, atol=1e-4)
    assert torch.allclose(ours(input_ids=ids).logits, want.logits, atol=1e-3)
    assert GPT2LMHeadModel.module_names(ours.config)[:4] == ["transformer.wte", "transformer.wpe", "transformer.drop", "transformer.h.0"]
    got.loss.backward()
    want.loss.backward()
    a = ours.transformer.h[0].attn.c_attn.weight.grad
    b = hf.transformer.h[0].attn.c_attn.weight.grad
    assert torch.allclose(a, b, atol=1e-4)


def test_bert_matches_hf():
    from transformers import BertConfig as HC, BertForMaskedLM as HM

    from cornstarch_b200.models.text_legacy import BertConfig, BertForMaskedLM

    kw = dict(num_hidden_layers=2, hidden_size=32, num_attention_heads=4, intermediate_size=64, vocab_size=100, max_position_embeddings=64)
    torch.manual_seed(0)
    hf = HM(HC(hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, **kw)).eval()
    ours = BertForMaskedLM(BertConfig(**kw)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (2, 20))
    am = torch.ones(2, 20, dtype=torch.long)
    am[1, 15:] = 0
    labels = torch.where(torch.rand(2, 20) < 0.3, ids, torch.full_like(ids, -100))
    labels[0, 0] = ids[0, 0]
    want = hf(input_ids=ids, attention_mask=am, labels=labels)
    got = ours(input_ids=ids, attention_mask=am, labels=labels)
    valid = am.bool()
    assert torch.allclose(got.logits[valid], want.logits[valid], atol=1e-3)
    assert BertForMaskedLM.module_names(ours.config) == ["bert.embeddings", "bert.encoder.layer.0", "bert.encoder.layer.1", "cls"]


def test_opt_matches_hf():
    from transformers import OPTConfig as HC, OPTForCausalLM as HM

    from cornstarch_b200.models.text_legacy import OPTConfig, OPTForCausalLM

    kw = dict(num_hidden_layers=2, hidden_size=32, num_attention_heads=4, ffn_dim=64, vocab_size=100, max_position_embeddings=64,
              word_embed_proj_dim=32)
    torch.manual_seed(0)
    hf = HM(HC(dropout=0.0, **kw)).eval()
    ours = OPTForCausalLM(OPTConfig(**kw)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (2, 24))
    want = hf(input_ids=ids, labels=ids)
    got = ours(input_ids=ids, labels=ids)
    assert torch.allclose(got.loss, want.loss, atol=1e-4)
    assert OPTForCausalLM.module_names(ours.config)[-2:] == ["model.decoder.final_layer_norm", "lm_head"]


def test_recompute_keeps_gradients():
    """Layer recomputation (activation checkpointing) yields the gradients of the plain forward."""
    from cornstarch_b200.models.text_legacy import GPT2Config, GPT2LMHeadModel

    torch.manual_seed(0)
    m = GPT2LMHeadModel(GPT2Config(n_layer=2, n_embd=32, n_head=4, vocab_size=100, n_positions=64))
    ids = torch.randint(0, 100, (2, 24))
    m(input_ids=ids, labels=ids).loss.backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    m.gradient_checkpointing_enable()
    m.train()
    m(input_ids=ids, labels=ids).loss.backward()
    for n, p in m.named_parameters():
        assert torch.allclose(p.grad, ref[n], atol=1e-6), n


def test_llama4_text_matches_hf():
    from transformers import Llama4TextConfig as HC
    from transformers.models.llama4.modeling_llama4 import Llama4ForCausalLM as HM

    from cornstarch_b200.models.llama4 import Llama4ForCausalLM, Llama4TextConfig

    kw = dict(vocab_size=100, hidden_size=32, intermediate_size=48, intermediate_size_mlp=64, num_hidden_layers=4,
              num_attention_heads=4, num_key_value_heads=2, head_dim=8, num_local_experts=4, num_experts_per_tok=1,
              interleave_moe_layer_step=2, max_position_embeddings=64, attention_chunk_size=64)
    torch.manual_seed(0)
    hfc = HC(**kw)
    hfc._attn_implementation = "eager"
    hf = HM(hfc).eval()
    ours = Llama4ForCausalLM(Llama4TextConfig(**kw, rope_theta=hfc.rope_parameters["rope_theta"] if getattr(hfc, "rope_parameters", None) else 500000.0)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (2, 24))
    want = hf(input_ids=ids, labels=ids)
    got = ours(input_ids=ids, labels=ids)
    assert torch.allclose(got.loss, want.loss, atol=1e-4), (got.loss, want.loss)
    assert torch.allclose(ours(input_ids=ids).logits, want.logits, atol=2e-3)
    assert Llama4ForCausalLM.module_names(ours.config)[:3] == ["model.embed_tokens", "model.rotary_emb", "model.layers.0"]
    assert ours.config.moe_layers == [1, 3] and ours.config.no_rope_layers == [1, 1, 1, 0]


def test_llama4_chunked_attention_matches_hf():
    """Sequences longer than ``attention_chunk_size``: RoPE layers attend causally inside chunks, NoPE layers over everything."""
    from transformers import Llama4TextConfig as HC
    from transformers.models.llama4.modeling_llama4 import Llama4ForCausalLM as HM

    from cornstarch_b200.models.llama4 import Llama4ForCausalLM, Llama4TextConfig

    kw = dict(vocab_size=100, hidden_size=32, intermediate_size=48, intermediate_size_mlp=64, num_hidden_layers=4,
              num_attention_heads=4, num_key_value_heads=2, head_dim=8, num_local_experts=4, num_experts_per_tok=1,
              interleave_moe_layer_step=2, max_position_embeddings=128, attention_chunk_size=16)
    torch.manual_seed(0)
    hfc = HC(**kw)
    hfc._attn_implementation = "eager"
    hf = HM(hfc).eval()
    ours = Llama4ForCausalLM(Llama4TextConfig(**kw, rope_theta=hfc.rope_parameters["rope_theta"] if getattr(hfc, "rope_parameters", None) else 500000.0)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (2, 40))  # 2.5 chunks
    with torch.no_grad():
        want = hf(input_ids=ids).logits
        got = ours(input_ids=ids).logits
    assert torch.allclose(got, want, atol=2e-3), (got - want).abs().max()
