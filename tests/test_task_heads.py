"""Task-head models (BERT x7, GPT-2 x4, OPT x2, Llama sequence classification, DINOv2 backbone / classifier): the
``transformers`` state dict loads unchanged and logits / losses agree with the ``transformers`` forward (fp32, CPU); every
class has a registered policy whose pipeline units are the backbone's units plus the head units on the last stage."""

import pytest
import torch

tf = pytest.importorskip("transformers")

from cornstarch_b200.models import task_heads as H  # noqa: E402
from cornstarch_b200.models.llama import LlamaConfig  # noqa: E402
from cornstarch_b200.models.text_legacy import BertConfig, GPT2Config, OPTConfig  # noqa: E402
from cornstarch_b200.models.vision_extra import Dinov2Config  # noqa: E402
from cornstarch_b200.pipeline_template import PipelineTemplate  # noqa: E402
from cornstarch_b200.shardformer.policies.auto_policy import get_autopolicy, get_policy_type, policy_for_model  # noqa: E402

BERT = dict(num_hidden_layers=2, hidden_size=32, num_attention_heads=4, intermediate_size=64, vocab_size=100, max_position_embeddings=64)
GPT2 = dict(n_layer=2, n_embd=32, n_head=4, vocab_size=100, n_positions=64)
OPT = dict(num_hidden_layers=2, hidden_size=32, num_attention_heads=4, ffn_dim=64, vocab_size=100, max_position_embeddings=64,
           word_embed_proj_dim=32)


def _load(ours, hf):
    missing, unexpected = ours.load_state_dict(hf.state_dict(), strict=False)
    assert not [m for m in missing if "rotary" not in m], missing
    assert not unexpected, unexpected


def _close(a, b, tol=2e-4):
    assert torch.allclose(a.float(), b.float(), atol=tol, rtol=1e-3), (a.float() - b.float()).abs().max()


def _bert(name, **extra):
    torch.manual_seed(0)
    hf = getattr(tf, name)(tf.BertConfig(hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, **BERT, **extra)).eval()
    ours = getattr(H, name)(BertConfig(**BERT, **extra)).eval()
    _load(ours, hf)
    ids = torch.randint(0, 100, (3, 12))
    am = torch.ones(3, 12, dtype=torch.long)
    am[1, 9:] = 0
    tt = torch.zeros(3, 12, dtype=torch.long)
    tt[:, 6:] = 1
    return hf, ours, ids, am, tt


def test_bert_pretraining_and_nsp():
    hf, ours, ids, am, tt = _bert("BertForPreTraining")
    labels = torch.where(torch.rand(3, 12) < 0.3, ids, torch.full_like(ids, -100))
    labels[0, 0] = ids[0, 0]
    nsl = torch.tensor([0, 1, 0])
    want = hf(input_ids=ids, attention_mask=am, token_type_ids=tt, labels=labels, next_sentence_label=nsl)
    got = ours(input_ids=ids, attention_mask=am, token_type_ids=tt, labels=labels, next_sentence_label=nsl)
    _close(got.prediction_logits[am.bool()], want.prediction_logits[am.bool()], 1e-3)
    _close(got.seq_relationship_logits, want.seq_relationship_logits)
    _close(got.loss, want.loss, 1e-3)
    hf, ours, ids, am, tt = _bert("BertForNextSentencePrediction")
    want = hf(input_ids=ids, attention_mask=am, token_type_ids=tt, labels=nsl)
    got = ours(input_ids=ids, attention_mask=am, token_type_ids=tt, labels=nsl)
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    assert H.BertForPreTraining.module_names(ours.config) == ["bert.embeddings", "bert.encoder.layer.0", "bert.encoder.layer.1", "bert.pooler", "cls"]


def test_bert_lm_head_decoder():
    hf, ours, ids, am, tt = _bert("BertLMHeadModel", is_decoder=True)
    want = hf(input_ids=ids, labels=ids)
    got = ours(input_ids=ids, labels=ids)
    _close(got.logits, want.logits, 1e-3)
    _close(got.loss, want.loss, 1e-3)
    assert H.BertLMHeadModel.module_names(ours.config)[-2:] == ["bert.encoder.layer.1", "cls"]


def test_bert_classification_heads():
    hf, ours, ids, am, tt = _bert("BertForSequenceClassification", num_labels=3)
    y = torch.tensor([0, 2, 1])
    want, got = hf(input_ids=ids, attention_mask=am, labels=y), ours(input_ids=ids, attention_mask=am, labels=y)
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    assert H.BertForSequenceClassification.module_names(ours.config)[-3:] == ["bert.pooler", "dropout", "classifier"]
    hf, ours, ids, am, tt = _bert("BertForTokenClassification", num_labels=5)
    y = torch.randint(0, 5, (3, 12))
    want, got = hf(input_ids=ids, attention_mask=am, labels=y), ours(input_ids=ids, attention_mask=am, labels=y)
    _close(got.logits[am.bool()], want.logits[am.bool()])
    assert H.BertForTokenClassification.module_names(ours.config)[-3:] == ["bert.encoder.layer.1", "dropout", "classifier"]
    hf, ours, ids, am, tt = _bert("BertForMultipleChoice")
    ids4 = torch.randint(0, 100, (2, 4, 10))
    y = torch.tensor([1, 3])
    want, got = hf(input_ids=ids4, labels=y), ours(input_ids=ids4, labels=y)
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    hf, ours, ids, am, tt = _bert("BertForQuestionAnswering")
    sp, ep = torch.tensor([1, 3, 5]), torch.tensor([4, 7, 30])  # the last end position lies outside the sequence: ignored
    want = hf(input_ids=ids, attention_mask=am, start_positions=sp, end_positions=ep)
    got = ours(input_ids=ids, attention_mask=am, start_positions=sp, end_positions=ep)
    _close(got.start_logits[am.bool()], want.start_logits[am.bool()])
    _close(got.end_logits[am.bool()], want.end_logits[am.bool()])
    assert H.BertForQuestionAnswering.module_names(ours.config)[-1] == "qa_outputs"


def _gpt2(name, **extra):
    torch.manual_seed(0)
    hf = getattr(tf, name)(tf.GPT2Config(resid_pdrop=0, embd_pdrop=0, attn_pdrop=0, summary_first_dropout=0.0, **GPT2, **extra)).eval()
    ours = getattr(H, name)(GPT2Config(**GPT2, **extra)).eval()
    _load(ours, hf)
    return hf, ours


def test_gpt2_heads():
    hf, ours = _gpt2("GPT2DoubleHeadsModel", num_labels=1)
    ids = torch.randint(0, 100, (2, 3, 10))
    mc_ids = torch.tensor([[9, 5, 7], [3, 9, 8]])
    want = hf(input_ids=ids, mc_token_ids=mc_ids, labels=ids, mc_labels=torch.tensor([0, 2]))
    got = ours(input_ids=ids, mc_token_ids=mc_ids, labels=ids, mc_labels=torch.tensor([0, 2]))
    _close(got.logits, want.logits, 1e-3)
    _close(got.mc_logits, want.mc_logits)
    _close(got.loss, want.loss, 1e-3)
    _close(got.mc_loss, want.mc_loss)
    assert H.GPT2DoubleHeadsModel.module_names(ours.config)[-3:] == ["transformer.ln_f", "lm_head", "multiple_choice_head"]
    hf, ours = _gpt2("GPT2ForSequenceClassification", num_labels=3, pad_token_id=0)
    ids = torch.randint(1, 100, (3, 12))
    ids[1, 8:] = 0
    want, got = hf(input_ids=ids, labels=torch.tensor([0, 1, 2])), ours(input_ids=ids, labels=torch.tensor([0, 1, 2]))
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    hf, ours = _gpt2("GPT2ForTokenClassification", num_labels=4, classifier_dropout=0.0)
    y = torch.randint(0, 4, (3, 12))
    want, got = hf(input_ids=ids, labels=y), ours(input_ids=ids, labels=y)
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    hf, ours = _gpt2("GPT2ForQuestionAnswering")
    want = hf(input_ids=ids, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    got = ours(input_ids=ids, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    _close(got.start_logits, want.start_logits)
    _close(got.loss, want.loss)


def test_opt_heads():
    torch.manual_seed(0)
    hf = tf.OPTForSequenceClassification(tf.OPTConfig(dropout=0.0, num_labels=3, pad_token_id=1, **OPT)).eval()
    ours = H.OPTForSequenceClassification(OPTConfig(num_labels=3, pad_token_id=1, **OPT)).eval()
    _load(ours, hf)
    ids = torch.randint(2, 100, (3, 12))
    am = torch.ones_like(ids)
    ids[2, 7:] = 1
    am[2, 7:] = 0
    want = hf(input_ids=ids, attention_mask=am, labels=torch.tensor([2, 0, 1]))
    got = ours(input_ids=ids, attention_mask=am, labels=torch.tensor([2, 0, 1]))
    _close(got.logits, want.logits)
    _close(got.loss, want.loss)
    assert H.OPTForSequenceClassification.module_names(ours.config)[-2:] == ["model.decoder.final_layer_norm", "score"]
    hf = tf.OPTForQuestionAnswering(tf.OPTConfig(dropout=0.0, **OPT)).eval()
    ours = H.OPTForQuestionAnswering(OPTConfig(**OPT)).eval()
    _load(ours, hf)
    want = hf(input_ids=ids, attention_mask=am, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    got = ours(input_ids=ids, attention_mask=am, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    _close(got.start_logits[am.bool()], want.start_logits[am.bool()])
    # the span loss normalises over every position, padded ones included, whose hidden states are arbitrary: compare it unpadded
    full = torch.randint(2, 100, (3, 12))
    want = hf(input_ids=full, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    got = ours(input_ids=full, start_positions=torch.tensor([1, 2, 3]), end_positions=torch.tensor([4, 5, 6]))
    _close(got.loss, want.loss)


def test_llama_sequence_classification():
    kw = dict(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              max_position_embeddings=64)
    torch.manual_seed(0)
    hf = tf.LlamaForSequenceClassification(tf.LlamaConfig(num_labels=3, pad_token_id=0, **kw)).eval()
    ours = H.LlamaForSequenceClassification(LlamaConfig(num_labels=3, pad_token_id=0, **kw)).eval()
    _load(ours, hf)
    ids = torch.randint(1, 100, (3, 12))
    ids[0, 9:] = 0
    want, got = hf(input_ids=ids, labels=torch.tensor([1, 0, 2])), ours(input_ids=ids, labels=torch.tensor([1, 0, 2]))
    _close(got.logits, want.logits, 1e-3)
    _close(got.loss, want.loss, 1e-3)
    names = H.LlamaForSequenceClassification.module_names(ours.config)
    assert names[0] == "model.embed_tokens" and names[-2:] == ["model.norm", "score"]


def test_dinov2_backbone_and_classifier():
    kw = dict(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)
    torch.manual_seed(0)
    hf = tf.Dinov2ForImageClassification(tf.Dinov2Config(num_labels=5, hidden_dropout_prob=0.0, **kw)).eval()
    ours = H.Dinov2ForImageClassification(Dinov2Config(num_labels=5, **kw)).eval()
    _load(ours, hf)
    pix = torch.randn(2, 3, 28, 28)
    y = torch.tensor([4, 1])
    want, got = hf(pixel_values=pix, labels=y), ours(pixel_values=pix, labels=y)
    _close(got.logits, want.logits, 1e-3)
    _close(got.loss, want.loss, 1e-3)
    assert H.Dinov2ForImageClassification.module_names(ours.config) == [
        "dinov2.embeddings", "dinov2.encoder.layer.0", "dinov2.encoder.layer.1", "dinov2.layernorm", "classifier"]
    hfb = tf.Dinov2Backbone(tf.Dinov2Config(hidden_dropout_prob=0.0, **kw)).eval()
    oursb = H.Dinov2Backbone(Dinov2Config(**kw)).eval()
    _load(oursb, hfb)
    _close(oursb(pixel_values=pix).feature_maps[0], hfb(pixel_values=pix).feature_maps[0], 1e-3)
    assert H.Dinov2Backbone.module_names(oursb.config) == ["embeddings", "encoder.layer.0", "encoder.layer.1", "layernorm"]


REFERENCE_NAMES = {
    "transformers.models.bert.modeling_bert.BertForPreTraining": H.BertForPreTraining,
    "transformers.models.bert.modeling_bert.BertLMHeadModel": H.BertLMHeadModel,
    "transformers.models.bert.modeling_bert.BertForSequenceClassification": H.BertForSequenceClassification,
    "transformers.models.bert.modeling_bert.BertForTokenClassification": H.BertForTokenClassification,
    "transformers.models.bert.modeling_bert.BertForNextSentencePrediction": H.BertForNextSentencePrediction,
    "transformers.models.bert.modeling_bert.BertForMultipleChoice": H.BertForMultipleChoice,
    "transformers.models.bert.modeling_bert.BertForQuestionAnswering": H.BertForQuestionAnswering,
    "transformers.models.llama.modeling_llama.LlamaForSequenceClassification": H.LlamaForSequenceClassification,
    "transformers.models.gpt2.modeling_gpt2.GPT2DoubleHeadsModel": H.GPT2DoubleHeadsModel,
    "transformers.models.gpt2.modeling_gpt2.GPT2ForQuestionAnswering": H.GPT2ForQuestionAnswering,
    "transformers.models.gpt2.modeling_gpt2.GPT2ForTokenClassification": H.GPT2ForTokenClassification,
    "transformers.models.gpt2.modeling_gpt2.GPT2ForSequenceClassification": H.GPT2ForSequenceClassification,
    "transformers.models.opt.modeling_opt.OPTForSequenceClassification": H.OPTForSequenceClassification,
    "transformers.models.opt.modeling_opt.OPTForQuestionAnswering": H.OPTForQuestionAnswering,
    "transformers.models.dinov2.modeling_dinov2.Dinov2ForImageClassification": H.Dinov2ForImageClassification,
    "transformers.models.dinov2.modeling_dinov2.Dinov2Backbone": H.Dinov2Backbone,
}


def test_every_head_has_a_policy_and_a_two_stage_template():
    cfgs = {"Bert": BertConfig(**BERT), "GPT2": GPT2Config(**GPT2), "OPTF": OPTConfig(**OPT),
            "Llam": LlamaConfig(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                num_key_value_heads=2),
            "Dino": Dinov2Config(hidden_size=32, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14)}
    for name, cls in REFERENCE_NAMES.items():
        pol_cls = get_policy_type(name)
        assert pol_cls.model_cls is cls, name
        cfg = cfgs[{"Deco": "Llam"}.get(cls.__name__[:4], cls.__name__[:4])]
        model = cls(cfg)
        pol = policy_for_model(model)
        assert type(pol) is pol_cls
        units = pol_cls.get_all_modules(cfg)
        assert units == cls.module_names(cfg)
        # the head units must sit on the last stage: a template that ends the first stage after the head is refused
        k = len(units) - len([u for u in pol.last_stage_modules if u in units])
        cut = max(1, min(4, k))
        good = PipelineTemplate(cls.__name__, [units[:cut], units[cut:]])
        pol.pipeline_template_sanity_check(good)
        bad = PipelineTemplate(cls.__name__, [units[:-1][:1] + units[-1:], units[1:-1]])
        with pytest.raises(ValueError):
            pol.pipeline_template_sanity_check(bad)
    assert get_autopolicy("transformers.models.qwen2_vl.modeling_qwen2_vl.Qwen2VLForConditionalGeneration") is not None


def test_modal_module_policy_units_and_sharding():
    from cornstarch_b200.shardformer.policies.multimodal import ModalModulePolicy
    from cornstarch_b200.zoo import build_model

    model = build_model("tiny")
    enc = model.vision_encoder
    for name in ("cornstarch.models.multimodal_language_model.modeling_multimodal_language_model.ModalEncoderModule",
                 "cornstarch.models.multimodal_language_model.modeling_multimodal_language_model.ModalDecoderModule"):
        assert get_policy_type(name) is ModalModulePolicy
    pol = policy_for_model(enc)
    assert isinstance(pol, ModalModulePolicy)
    units = pol.all_modules()
    assert units[0] == "module.embeddings" and units[-1].startswith("projector.")
    pol.pipeline_template_sanity_check(PipelineTemplate("vision", [units[:2], units[2:]]))
    with pytest.raises(ValueError):
        pol.pipeline_template_sanity_check(PipelineTemplate("vision", [units[:1] + units[-1:], units[1:-1]]))
