"""``ShardFormer``: apply a policy to a model — keep only the held pipeline units, convert projections to
tensor-parallel layers, divide head counts, attach the parallel context.

Order of operations (same contract as cornstarch/shardformer/shard/shardformer.py:22-45 in the
reference): replace modules -> release unheld layers -> materialise what is left.  Released parameters
are remembered as :class:`TensorPlaceholder` records so the same model object can be re-sharded after a
re-plan (``ModelSharder.set_tensors_to_placeholder`` in the reference, :47-111).
"""

from __future__ import annotations

import re

import torch
import torch.distributed as dist
import torch.nn as nn

from ... import nn as cnn
from ...models.base import PreTrainedModel
from ...models.llama import ParallelContext
from .placeholder import TensorPlaceholder
from .shard_config import ShardConfig


def _get_submodule(root: nn.Module, path: str):
    obj = root
    for p in path.split("."):
        obj = obj[int(p)] if p.isdigit() else getattr(obj, p)
    return obj


def _set_submodule(root: nn.Module, path: str, new: nn.Module):
    parts = path.split(".")
    parent = _get_submodule(root, ".".join(parts[:-1])) if len(parts) > 1 else root
    last = parts[-1]
    if last.isdigit():
        parent[int(last)] = new
    else:
        setattr(parent, last, new)


class ModelSharder:
    def __init__(self, model: nn.Module, policy, shard_config: ShardConfig):
        self.model, self.policy, self.shard_config = model, policy, shard_config
        self.placeholders: dict[str, TensorPlaceholder] = {}

    def shard(self) -> list[dict]:
        self.policy.set_model(self.model)
        self.policy.set_shard_config(self.shard_config)
        self.policy.config_sanity_check()
        self._release_unheld()
        self._replace_tp()
        self._attach_context()
        self._materialize()
        return self.policy.get_shared_params()

    # ---- pipeline: keep only the held units
    def _release_unheld(self):
        sm = self.shard_config.pipeline_stage_manager
        if sm is None or not isinstance(self.model, PreTrainedModel):
            return
        template = self.shard_config.pipeline_template
        if template is not None:
            self.policy.pipeline_template_sanity_check(template)
        held = self.policy.get_held_layers()
        all_names = type(self.policy).get_all_modules(self.model.config)
        for name in all_names:
            if name in held:
                continue
            try:
                mod = _get_submodule(self.model, name)
            except (AttributeError, IndexError):
                continue
            if isinstance(mod, nn.Module):
                for pn, p in mod.named_parameters():
                    self.placeholders[f"{name}.{pn}"] = TensorPlaceholder(p)
        self.model.hold_only(held)

    # ---- tensor parallelism
    def _replace_tp(self):
        sc = self.shard_config
        tp_group = sc.tensor_parallel_process_group
        tp = sc.tensor_parallel_size
        if tp <= 1:
            return
        rules = [(re.compile(r.pattern), r) for r in self.policy.tp_rules]
        from ...models.text_legacy import Conv1D

        # parameters that several modules share (tie_word_embeddings: embed_tokens.weight is lm_head.weight): each
        # tensor-parallel layer below takes its own copy of its shard, so the ties are restored afterwards
        owners: dict[int, list[tuple[str, str]]] = {}
        for path, mod in self.model.named_modules():
            for pn, prm in mod._parameters.items():
                if prm is not None:
                    owners.setdefault(id(prm), []).append((path, pn))
        tied = [v for v in owners.values() if len(v) > 1]

        for path, mod in list(self.model.named_modules()):
            if isinstance(mod, Conv1D) and mod.parallel is None:
                for rx, rule in rules:
                    if rx.fullmatch(path):
                        _set_submodule(self.model, path, Conv1D.shard(mod, tp_group, rule.kind, self.policy.split_sizes(path, mod)))
                        break
                continue
            if not isinstance(mod, (cnn.Linear, cnn.Embedding)) or isinstance(
                    mod, (cnn.ColumnParallelLinear, cnn.RowParallelLinear, cnn.VocabParallelEmbedding)):
                continue
            for rx, rule in rules:
                if not rx.fullmatch(path):
                    continue
                if rule.kind in ("col", "col_gather"):
                    new = cnn.ColumnParallelLinear.from_native_module(
                        mod, tp_group, gather_output=(rule.kind == "col_gather"), split_sizes=self.policy.split_sizes(path, mod))
                elif rule.kind == "row":
                    new = cnn.RowParallelLinear.from_native_module(mod, tp_group, split_sizes=self.policy.split_sizes(path, mod))
                elif rule.kind == "vocab":
                    new = cnn.VocabParallelEmbedding.from_native_module(mod, tp_group, sc.make_vocab_size_divisible_by)
                elif rule.kind == "lm_head":
                    new = self._shard_lm_head(mod, tp_group, tp)
                else:
                    raise ValueError(rule.kind)
                _set_submodule(self.model, path, new)
                break
        for group in tied:
            # the vocabulary padding and the row split of the embedding and the LM head are identical, so the shards
            # of a tied pair have the same shape and hold the same rows: one Parameter again
            (path0, pn0), rest = group[0], group[1:]
            first = _get_submodule(self.model, path0)._parameters.get(pn0) if path0 else self.model._parameters.get(pn0)
            for path, pn in rest:
                mod = _get_submodule(self.model, path) if path else self.model
                other = mod._parameters.get(pn)
                if first is not None and other is not None and other is not first and other.shape == first.shape:
                    mod._parameters[pn] = first
        if self.policy.head_modules:
            rx = re.compile(self.policy.head_modules)
            for path, mod in self.model.named_modules():
                if rx.fullmatch(path):
                    for attr in ("num_heads", "num_kv_heads"):
                        if hasattr(mod, attr) and not getattr(mod, "_tp_divided", False):
                            setattr(mod, attr, getattr(mod, attr) // tp)
                    mod._tp_divided = True

    def _shard_lm_head(self, mod: cnn.Linear, tp_group, tp: int):
        """Vocab-parallel LM head: rows padded to a multiple of ``divisible_by * tp`` and split across ranks."""
        V, H = mod.weight.shape
        mult = self.shard_config.make_vocab_size_divisible_by * tp
        Vp = (V + mult - 1) // mult * mult
        w = mod.weight.data
        if Vp != V:
            w = torch.cat([w, w.new_zeros(Vp - V, H)], dim=0)
        r = dist.get_rank(tp_group)
        local = Vp // tp
        new = cnn.ColumnParallelLinear(H, Vp, bias=False, process_group=tp_group, device="meta", dtype=w.dtype)
        new.weight = nn.Parameter(w[r * local : (r + 1) * local].clone(), requires_grad=mod.weight.requires_grad)
        new.full_vocab_size = V
        new.vocab_start = r * local
        new.valid_rows = max(0, min(local, V - r * local))
        if hasattr(self.model, "vocab_start"):
            self.model.vocab_start = new.vocab_start
            self.model.valid_vocab = new.valid_rows
        return new

    # ---- context
    def _attach_context(self):
        sc = self.shard_config
        pc = ParallelContext(
            tp_group=sc.tensor_parallel_process_group if sc.enable_tensor_parallelism else None,
            sp_group=sc.sequence_parallel_process_group if sc.enable_sequence_parallelism else None,
            sp_mode=sc.sequence_parallelism_mode if sc.enable_sequence_parallelism else None,
            cp_dist_mode=sc.context_parallel_distribution_mode, parallel_output=sc.parallel_output,
            tp_seq_shard=sc.tensor_parallel_sequence_sharding)
        if hasattr(self.model, "set_parallel_context"):
            self.model.set_parallel_context(pc)
        else:
            self.model.pc = pc
        if pc.sp_mode == "ring_attn" and pc.sp_size > 1:
            from ...parallel.cp import install_context_parallel_attention

            install_context_parallel_attention(self.model, pc.sp_group)

    def _materialize(self):
        """Give real storage to parameters that were built on the meta device (lazy construction)."""
        device = self.shard_config.extra_kwargs.get("device")
        dtype = self.shard_config.extra_kwargs.get("dtype")
        materialize_meta(self.model, device, dtype)


def materialize_meta(module: nn.Module, device=None, dtype=None, std: float = 0.02) -> None:
    """Allocate and initialise every meta parameter/buffer of ``module`` (normal(0, std) matrices, unit norm weights, zero biases)."""
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    for mod in module.modules():
        for name, p in list(mod._parameters.items()):
            if p is None or p.device.type != "meta":
                continue
            t = torch.empty(p.shape, dtype=dtype or p.dtype, device=device)
            if p.dim() >= 2:
                t.normal_(0.0, std)
            elif name == "weight":
                t.fill_(0.0 if getattr(mod, "weight_offset", 0.0) else 1.0)
            else:
                t.zero_()
            mod._parameters[name] = nn.Parameter(t, requires_grad=p.requires_grad)
        for name, b in list(mod._buffers.items()):
            if b is not None and b.device.type == "meta":
                mod._buffers[name] = torch.zeros(b.shape, dtype=b.dtype, device=device)


class ShardFormer:
    """``ShardFormer(shard_config).optimize(model, policy)`` -> ``(model, shared_params)``."""

    def __init__(self, shard_config: ShardConfig):
        self.shard_config = shard_config

    def optimize(self, model: nn.Module, policy=None):
        if policy is None:
            from ..policies.auto_policy import policy_for_model

            policy = policy_for_model(model)
        if getattr(policy, "is_modal_module_policy", False):
            # a modality wrapper (encoder / decoder + projector): its parts are sharded by their own policies
            policy.set_model(model)
            policy.set_shard_config(self.shard_config)
            policy.shard(self.shard_config)
            return model, []
        sharder = ModelSharder(model, policy, self.shard_config)
        shared = sharder.shard()
        model._sharder_placeholders = sharder.placeholders
        ep_group = self.shard_config.expert_parallel_process_group
        if ep_group is not None and dist.get_world_size(ep_group) > 1:
            # experts of the sparse blocks that survived the pipeline cut are sharded over the expert-parallel group
            # (blocks that already are stay as they are); ``extra_kwargs["expert_capacity_factor"]`` selects capacity mode
            from ...parallel.ep import shard_experts

            shard_experts(model, ep_group, capacity_factor=self.shard_config.extra_kwargs.get("expert_capacity_factor"),
                          capacity_tokens=self.shard_config.extra_kwargs.get("expert_capacity_tokens"))
        return model, shared
