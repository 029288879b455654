"""Task heads over the BERT, GPT-2, OPT, Llama and DINOv2 backbones, with Hugging Face parameter names.

The reference registers a sharding policy for each of these classes (cornstarch/shardformer/policies/auto_policy.py:23-147:
seven BERT heads, four GPT-2 heads, two OPT heads, ``LlamaForSequenceClassification``, ``Dinov2Backbone``,
``Dinov2ForImageClassification``) and patches the ``transformers`` forwards; here every class is a thin native module
around the backbone of this package.  ``module_names`` lists the pipeline units the reference's ``get_all_modules``
returns for the class (policies/bert.py:106-260, policies/gpt2.py:97-180, policies/opt.py:99-135,
policies/dinov2.py:254-259): the backbone's units under its attribute prefix, then the head units in forward order.

A stage that does not hold the head returns ``hidden_states`` for the next stage, like every other model here.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import nn as cnn
from .base import ModelOutput, PreTrainedModel, is_released
from .llama import DecoderConfig, DecoderModel
from .text_legacy import BertConfig, BertModel, GPT2Config, GPT2Model, OPTConfig, OPTModel, _BertMLMHead, _BertPredictions
from .vision_extra import Dinov2Config, Dinov2Model


# ------------------------------------------------------------------------------------------------ helpers
def _classification_loss(logits, labels, num_labels: int, problem_type: str | None = None):
    """Regression for one label, cross-entropy for integer labels, BCE for multi-hot float labels (the HF convention)."""
    if problem_type is None:
        if num_labels == 1:
            problem_type = "regression"
        elif labels.dtype in (torch.long, torch.int):
            problem_type = "single_label_classification"
        else:
            problem_type = "multi_label_classification"
    lf = logits.float()
    if problem_type == "regression":
        return F.mse_loss(lf.squeeze(-1) if num_labels == 1 else lf, labels.float().squeeze(-1) if num_labels == 1 else labels.float())
    if problem_type == "single_label_classification":
        return F.cross_entropy(lf.view(-1, num_labels), labels.view(-1))
    return F.binary_cross_entropy_with_logits(lf, labels.float())


def _span_loss(logits, start_positions, end_positions):
    """Extractive question answering: mean of the start and end cross-entropies; positions outside the sequence are ignored."""
    start, end = logits.float().unbind(dim=-1)
    S = start.shape[1]
    sp, ep = start_positions.view(-1).clamp(0, S), end_positions.view(-1).clamp(0, S)
    return (F.cross_entropy(start, sp, ignore_index=S) + F.cross_entropy(end, ep, ignore_index=S)) / 2, start, end


def _last_token_index(input_ids, pad_token_id, S, device):
    """Index of the last non-padding token of every row (the whole row when there is no padding token)."""
    if pad_token_id is None or input_ids is None:
        return torch.full((1,), S - 1, dtype=torch.long, device=device)
    non_pad = (input_ids != pad_token_id).to(torch.int32)
    return (torch.arange(S, device=input_ids.device, dtype=torch.int32) * non_pad).argmax(-1).to(device)


class _HeadModel(PreTrainedModel):
    """Backbone under ``self.<prefix>`` plus head units; subclasses implement ``_head(out, **kw)``."""

    prefix = ""
    head_units: list[str] = []
    backbone_kwargs: dict = {}

    @classmethod
    def _backbone_names(cls, config):
        raise NotImplementedError

    @classmethod
    def module_names(cls, config):
        return [f"{cls.prefix}.{n}" for n in cls._backbone_names(config)] + list(cls.head_units)

    def _backbone(self):
        return getattr(self, self.prefix)

    def _holds_head(self) -> bool:
        return all(self.holds(u) for u in self.head_units)

    def get_input_embeddings(self):
        return self._backbone().get_input_embeddings() if hasattr(self._backbone(), "get_input_embeddings") else None

    def hold_only(self, names):
        super().hold_only(names)
        inner = self._backbone()
        if isinstance(inner, PreTrainedModel):
            inner._held = {n[len(self.prefix) + 1:] for n in names if n.startswith(self.prefix + ".")}


# ------------------------------------------------------------------------------------------------ BERT
class _BertHeadModel(_HeadModel):
    config_class = BertConfig
    prefix = "bert"
    pooling = True

    @classmethod
    def _backbone_names(cls, config):
        return BertModel.module_names(config, cls.pooling)

    def _run(self, input_ids, attention_mask, token_type_ids, hidden_states):
        self.bert.gradient_checkpointing = self.gradient_checkpointing
        out = self.bert(input_ids=input_ids, attention_mask=attention_mask, token_type_ids=token_type_ids, hidden_states=hidden_states)
        if "last_hidden_state" not in out or not self._holds_head():
            return None, ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        return out, None


class _BertPreTrainingHeads(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.predictions = _BertPredictions(config)
        self.seq_relationship = cnn.Linear(config.hidden_size, 2)


class BertForPreTraining(_BertHeadModel):
    """Masked-LM head + next-sentence head (``cls.predictions``, ``cls.seq_relationship``)."""

    head_units = ["cls"]

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=True)
        self.cls = _BertPreTrainingHeads(config)
        if config.tie_word_embeddings:
            self.cls.predictions.decoder.weight = self.bert.embeddings.word_embeddings.weight

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, next_sentence_label=None,
                hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        p = self.cls.predictions
        scores = F.linear(p.transform(out.last_hidden_state), p.decoder.weight, p.decoder.bias)
        rel = self.cls.seq_relationship(out.pooler_output)
        res = ModelOutput(prediction_logits=scores, seq_relationship_logits=rel)
        if labels is not None and next_sentence_label is not None:
            res["loss"] = (F.cross_entropy(scores.float().view(-1, scores.shape[-1]), labels.reshape(-1), ignore_index=-100)
                           + F.cross_entropy(rel.float().view(-1, 2), next_sentence_label.view(-1)))
        return res


class BertLMHeadModel(_BertHeadModel):
    """Next-token prediction with the masked-LM head (``cls``); attention is causal when ``config.is_decoder``."""

    head_units = ["cls"]
    pooling = False

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=False)
        self.cls = _BertMLMHead(config)
        if config.tie_word_embeddings:
            self.cls.predictions.decoder.weight = self.bert.embeddings.word_embeddings.weight

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        p = self.cls.predictions
        logits = F.linear(p.transform(out.last_hidden_state), p.decoder.weight, p.decoder.bias)
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = F.cross_entropy(logits[:, :-1].float().reshape(-1, logits.shape[-1]), labels[:, 1:].reshape(-1), ignore_index=-100)
        return res


class BertForSequenceClassification(_BertHeadModel):
    head_units = ["dropout", "classifier"]

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.bert = BertModel(config, add_pooling_layer=True)
        self.dropout = nn.Dropout(getattr(config, "classifier_dropout", None) or getattr(config, "hidden_dropout_prob", 0.0))
        self.classifier = cnn.Linear(config.hidden_size, self.num_labels)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        logits = self.classifier(self.dropout(out.pooler_output))
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = _classification_loss(logits, labels, self.num_labels, getattr(self.config, "problem_type", None))
        return res


class BertForTokenClassification(_BertHeadModel):
    head_units = ["dropout", "classifier"]
    pooling = False

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.bert = BertModel(config, add_pooling_layer=False)
        self.dropout = nn.Dropout(getattr(config, "classifier_dropout", None) or getattr(config, "hidden_dropout_prob", 0.0))
        self.classifier = cnn.Linear(config.hidden_size, self.num_labels)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        logits = self.classifier(self.dropout(out.last_hidden_state))
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = F.cross_entropy(logits.float().view(-1, self.num_labels), labels.view(-1), ignore_index=-100)
        return res


class _BertOnlyNSPHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.seq_relationship = cnn.Linear(config.hidden_size, 2)


class BertForNextSentencePrediction(_BertHeadModel):
    head_units = ["cls"]

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=True)
        self.cls = _BertOnlyNSPHead(config)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        logits = self.cls.seq_relationship(out.pooler_output)
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = F.cross_entropy(logits.float().view(-1, 2), labels.view(-1))
        return res


class BertForMultipleChoice(_BertHeadModel):
    """Inputs are ``[batch, choices, seq]``; every choice is scored by one logit from the pooled output."""

    head_units = ["dropout", "classifier"]

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=True)
        self.dropout = nn.Dropout(getattr(config, "classifier_dropout", None) or getattr(config, "hidden_dropout_prob", 0.0))
        self.classifier = cnn.Linear(config.hidden_size, 1)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, labels=None, hidden_states=None, num_choices=None, **kw):
        if input_ids is not None:
            num_choices = input_ids.shape[1]
        flat = lambda t: None if t is None else t.reshape(-1, t.shape[-1])  # noqa: E731
        out, early = self._run(flat(input_ids), flat(attention_mask), flat(token_type_ids), hidden_states)
        if early is not None:
            return early
        logits = self.classifier(self.dropout(out.pooler_output)).view(-1, num_choices)
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = F.cross_entropy(logits.float(), labels.view(-1))
        return res


class BertForQuestionAnswering(_BertHeadModel):
    head_units = ["qa_outputs"]
    pooling = False

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config, add_pooling_layer=False)
        self.qa_outputs = cnn.Linear(config.hidden_size, 2)

    def forward(self, input_ids=None, attention_mask=None, token_type_ids=None, start_positions=None, end_positions=None,
                hidden_states=None, **kw):
        out, early = self._run(input_ids, attention_mask, token_type_ids, hidden_states)
        if early is not None:
            return early
        logits = self.qa_outputs(out.last_hidden_state)
        res = ModelOutput(start_logits=logits[..., 0], end_logits=logits[..., 1])
        if start_positions is not None and end_positions is not None:
            res["loss"], _, _ = _span_loss(logits, start_positions, end_positions)
        return res


# ------------------------------------------------------------------------------------------------ GPT-2
class _GPT2HeadModel(_HeadModel):
    config_class = GPT2Config
    prefix = "transformer"

    @classmethod
    def _backbone_names(cls, config):
        return GPT2Model.module_names(config)

    def _run(self, input_ids, attention_mask, hidden_states, **kw):
        self.transformer.gradient_checkpointing = self.gradient_checkpointing
        out = self.transformer(input_ids=input_ids, attention_mask=attention_mask, hidden_states=hidden_states, **kw)
        if "last_hidden_state" not in out or not self._holds_head():
            return None, ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        return out.last_hidden_state, None


class _SequenceSummary(nn.Module):
    """``summary``: one logit from the hidden state at a chosen token of every choice."""

    def __init__(self, config):
        super().__init__()
        self.summary = cnn.Linear(config.n_embd, 1)

    def forward(self, h, cls_index=None):
        if cls_index is None:
            picked = h[..., -1, :]
        else:
            idx = cls_index[..., None, None].expand(*cls_index.shape, 1, h.shape[-1])
            picked = h.gather(-2, idx).squeeze(-2)
        return self.summary(picked)


class GPT2DoubleHeadsModel(_GPT2HeadModel):
    """Language-model head + multiple-choice head; inputs are ``[batch, choices, seq]``."""

    head_units = ["lm_head", "multiple_choice_head"]

    def __init__(self, config):
        super().__init__(config)
        self.transformer = GPT2Model(config)
        self.lm_head = cnn.Linear(config.n_embd, config.vocab_size, bias=False)
        self.multiple_choice_head = _SequenceSummary(config)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.transformer.wte.weight

    def forward(self, input_ids=None, attention_mask=None, mc_token_ids=None, labels=None, mc_labels=None, hidden_states=None, **kw):
        shape = input_ids.shape if input_ids is not None else None
        flat = lambda t: None if t is None else t.reshape(-1, t.shape[-1])  # noqa: E731
        h, early = self._run(flat(input_ids), flat(attention_mask), hidden_states)
        if early is not None:
            return early
        if shape is not None and len(shape) == 3:
            h = h.view(shape[0], shape[1], shape[2], -1)
        lm_logits = self.lm_head(h)
        mc_logits = self.multiple_choice_head(h, mc_token_ids).squeeze(-1)
        res = ModelOutput(logits=lm_logits, mc_logits=mc_logits)
        if mc_labels is not None:
            res["mc_loss"] = F.cross_entropy(mc_logits.float().view(-1, mc_logits.shape[-1]), mc_labels.view(-1))
        if labels is not None:
            res["loss"] = F.cross_entropy(lm_logits[..., :-1, :].float().reshape(-1, lm_logits.shape[-1]), labels[..., 1:].reshape(-1),
                                          ignore_index=-100)
        return res


class GPT2ForQuestionAnswering(_GPT2HeadModel):
    head_units = ["qa_outputs"]

    def __init__(self, config):
        super().__init__(config)
        self.transformer = GPT2Model(config)
        self.qa_outputs = cnn.Linear(config.n_embd, 2)

    def forward(self, input_ids=None, attention_mask=None, start_positions=None, end_positions=None, hidden_states=None, **kw):
        h, early = self._run(input_ids, attention_mask, hidden_states)
        if early is not None:
            return early
        logits = self.qa_outputs(h)
        res = ModelOutput(start_logits=logits[..., 0], end_logits=logits[..., 1])
        if start_positions is not None and end_positions is not None:
            res["loss"], _, _ = _span_loss(logits, start_positions, end_positions)
        return res


class GPT2ForTokenClassification(_GPT2HeadModel):
    head_units = ["dropout", "classifier"]

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.transformer = GPT2Model(config)
        self.dropout = nn.Dropout(getattr(config, "classifier_dropout", None) or 0.0)
        self.classifier = cnn.Linear(config.n_embd, self.num_labels)

    def forward(self, input_ids=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        h, early = self._run(input_ids, attention_mask, hidden_states)
        if early is not None:
            return early
        logits = self.classifier(self.dropout(h))
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = F.cross_entropy(logits.float().view(-1, self.num_labels), labels.view(-1), ignore_index=-100)
        return res


class GPT2ForSequenceClassification(_GPT2HeadModel):
    """``score`` (no bias) applied to the hidden state of the last non-padding token."""

    head_units = ["score"]

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.transformer = GPT2Model(config)
        self.score = cnn.Linear(config.n_embd, self.num_labels, bias=False)

    def forward(self, input_ids=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        h, early = self._run(input_ids, attention_mask, hidden_states)
        if early is not None:
            return early
        logits = self.score(h)
        last = _last_token_index(input_ids, getattr(self.config, "pad_token_id", None), h.shape[1], h.device)
        pooled = logits[torch.arange(h.shape[0], device=h.device), last.expand(h.shape[0]) if last.numel() == 1 else last]
        res = ModelOutput(logits=pooled)
        if labels is not None:
            res["loss"] = _classification_loss(pooled, labels, self.num_labels, getattr(self.config, "problem_type", None))
        return res


# ------------------------------------------------------------------------------------------------ OPT
class _OPTHeadModel(_HeadModel):
    config_class = OPTConfig
    prefix = "model"

    @classmethod
    def _backbone_names(cls, config):
        return OPTModel.module_names(config)

    def _run(self, input_ids, attention_mask, hidden_states):
        self.model.gradient_checkpointing = self.gradient_checkpointing
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, hidden_states=hidden_states)
        if "last_hidden_state" not in out or not self._holds_head():
            return None, ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        return out.last_hidden_state, None

    def get_input_embeddings(self):
        return self.model.decoder.embed_tokens


class OPTForSequenceClassification(_OPTHeadModel):
    head_units = ["score"]

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.model = OPTModel(config)
        self.score = cnn.Linear(config.word_embed_proj_dim or config.hidden_size, self.num_labels, bias=False)

    def forward(self, input_ids=None, attention_mask=None, labels=None, hidden_states=None, **kw):
        h, early = self._run(input_ids, attention_mask, hidden_states)
        if early is not None:
            return early
        logits = self.score(h)
        last = _last_token_index(input_ids, getattr(self.config, "pad_token_id", None), h.shape[1], h.device)
        pooled = logits[torch.arange(h.shape[0], device=h.device), last.expand(h.shape[0]) if last.numel() == 1 else last]
        res = ModelOutput(logits=pooled)
        if labels is not None:
            res["loss"] = _classification_loss(pooled, labels, self.num_labels, getattr(self.config, "problem_type", None))
        return res


class OPTForQuestionAnswering(_OPTHeadModel):
    head_units = ["qa_outputs"]

    def __init__(self, config):
        super().__init__(config)
        self.model = OPTModel(config)
        self.qa_outputs = cnn.Linear(config.hidden_size, 2)

    def forward(self, input_ids=None, attention_mask=None, start_positions=None, end_positions=None, hidden_states=None, **kw):
        h, early = self._run(input_ids, attention_mask, hidden_states)
        if early is not None:
            return early
        logits = self.qa_outputs(h)
        res = ModelOutput(start_logits=logits[..., 0], end_logits=logits[..., 1])
        if start_positions is not None and end_positions is not None:
            res["loss"], _, _ = _span_loss(logits, start_positions, end_positions)
        return res


# ------------------------------------------------------------------------------------------------ Llama-style decoders
class DecoderForSequenceClassification(_HeadModel):
    """``LlamaForSequenceClassification`` (and the same head for every decoder family of this package): ``score`` on the
    last non-padding token."""

    config_class = DecoderConfig
    prefix = "model"
    head_units = ["score"]

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.model = DecoderModel(config)
        self.score = cnn.Linear(config.hidden_size, self.num_labels, bias=False)
        self.pc = None

    @classmethod
    def _backbone_names(cls, config):
        return DecoderModel.module_names(config)

    def hold_only(self, names):
        PreTrainedModel.hold_only(self, names)
        self.model._held = {n[len("model."):] for n in names if n.startswith("model.")}

    def set_parallel_context(self, pc):
        self.pc = pc
        self.model.set_parallel_context(pc)

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def forward(self, input_ids=None, inputs_embeds=None, attention_mask=None, position_ids=None, labels=None, hidden_states=None, **kw):
        self.model.gradient_checkpointing = self.gradient_checkpointing
        out = self.model(input_ids=input_ids, inputs_embeds=inputs_embeds, attention_mask=attention_mask, position_ids=position_ids,
                         hidden_states=hidden_states)
        h = out.last_hidden_state
        if not self.holds("score") or is_released(self.score):
            return ModelOutput(hidden_states=h)
        logits = self.score(h)
        last = _last_token_index(input_ids, getattr(self.config, "pad_token_id", None), h.shape[1], h.device)
        pooled = logits[torch.arange(h.shape[0], device=h.device), last.expand(h.shape[0]) if last.numel() == 1 else last]
        res = ModelOutput(logits=pooled)
        if labels is not None:
            res["loss"] = _classification_loss(pooled, labels, self.num_labels, getattr(self.config, "problem_type", None))
        return res


LlamaForSequenceClassification = DecoderForSequenceClassification


# ------------------------------------------------------------------------------------------------ DINOv2
class Dinov2Backbone(Dinov2Model):
    """Feature-map backbone: the final stage's tokens are normalised, the class token is dropped and the patch tokens
    are returned as a ``[B, hidden, h, w]`` map (the last stage of ``out_features``)."""

    @classmethod
    def module_names(cls, config):
        return ["embeddings"] + [f"encoder.layer.{i}" for i in range(config.num_hidden_layers)] + ["layernorm"]

    def forward(self, pixel_values=None, hidden_states=None, **kw):
        out = super().forward(pixel_values=pixel_values, hidden_states=hidden_states, **kw)
        if "last_hidden_state" not in out:
            return out
        x = out.last_hidden_state
        if getattr(self.config, "reshape_hidden_states", True):
            B, S, H = x.shape
            side = int(round((S - 1) ** 0.5))
            fmap = x[:, 1:].reshape(B, side, side, H).permute(0, 3, 1, 2).contiguous()
        else:
            fmap = x
        return ModelOutput(feature_maps=(fmap,), last_hidden_state=x)


class Dinov2ForImageClassification(_HeadModel):
    """``classifier`` over the class token concatenated with the mean of the patch tokens."""

    config_class = Dinov2Config
    prefix = "dinov2"
    head_units = ["classifier"]
    main_input_name = "pixel_values"

    def __init__(self, config):
        super().__init__(config)
        self.num_labels = getattr(config, "num_labels", 2)
        self.dinov2 = Dinov2Model(config)
        self.classifier = cnn.Linear(2 * config.hidden_size, self.num_labels)

    @classmethod
    def _backbone_names(cls, config):
        return Dinov2Model.module_names(config)

    def forward(self, pixel_values=None, labels=None, hidden_states=None, **kw):
        self.dinov2.gradient_checkpointing = self.gradient_checkpointing
        out = self.dinov2(pixel_values=pixel_values, hidden_states=hidden_states)
        if "last_hidden_state" not in out or not self._holds_head():
            return ModelOutput(hidden_states=out.get("hidden_states", out.get("last_hidden_state")))
        x = out.last_hidden_state
        logits = self.classifier(torch.cat([x[:, 0], x[:, 1:].mean(dim=1)], dim=1))
        res = ModelOutput(logits=logits)
        if labels is not None:
            res["loss"] = _classification_loss(logits, labels, self.num_labels, getattr(self.config, "problem_type", None))
        return res


__all__ = ["BertForPreTraining", "BertLMHeadModel", "BertForSequenceClassification", "BertForTokenClassification",
           "BertForNextSentencePrediction", "BertForMultipleChoice", "BertForQuestionAnswering", "GPT2DoubleHeadsModel",
           "GPT2ForQuestionAnswering", "GPT2ForTokenClassification", "GPT2ForSequenceClassification",
           "OPTForSequenceClassification", "OPTForQuestionAnswering", "DecoderForSequenceClassification",
           "LlamaForSequenceClassification", "Dinov2Backbone", "Dinov2ForImageClassification"]
