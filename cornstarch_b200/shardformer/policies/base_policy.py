"""Declarative sharding policies.

A policy names (a) the pipeline units of a model class, (b) which units must sit on the first / last
stage, and (c) a tensor-parallel plan: regular expressions over sub-module paths mapped to ``"col"``,
``"row"``, ``"vocab"`` or ``"lm_head"``, plus the attention modules whose head counts are divided by the
tp size.  :class:`~cornstarch_b200.shardformer.shard.shardformer.ShardFormer` applies it.  This replaces the
per-model ``module_policy()`` dictionaries of forward patches in the reference
(e.g. cornstarch/shardformer/policies/llama.py:96-347): the models here are pipeline- and TP-aware
natively, so a policy is data, not code.
"""

from __future__ import annotations

from dataclasses import dataclass

from .pipeline_template_policy import PipelineTemplatePolicyBase, check_template_covers


@dataclass
class TPRule:
    pattern: str  # regex matched against the dotted sub-module path (fullmatch)
    kind: str  # "col" | "row" | "vocab" | "lm_head" | "col_gather"
    split_sizes_attr: str | None = None  # for fused projections: attribute name on the policy computing split sizes


class ModelPolicy(PipelineTemplatePolicyBase):
    """Generic policy bound to a model class; subclasses fill the class attributes."""

    model_cls = None
    first_stage_modules: list[str] = []
    last_stage_modules: list[str] = []
    tp_rules: list[TPRule] = []
    head_modules: str | None = None  # regex of modules carrying num_heads / num_kv_heads attributes
    supported_sp_modes: tuple[str, ...] = ()

    def __init__(self):
        self.model = None
        self.shard_config = None

    @classmethod
    def get_all_modules(cls, config) -> list[str]:
        return cls.model_cls.module_names(config)

    def pipeline_template_sanity_check(self, template) -> None:
        cfg = self.model.config if self.model is not None else None
        assert cfg is not None, "set_model() first"
        check_template_covers(template, self.get_all_modules(cfg), self.first_stage_modules, self.last_stage_modules)

    def set_model(self, model):
        self.model = model

    def set_shard_config(self, shard_config):
        self.shard_config = shard_config

    def config_sanity_check(self):
        sc = self.shard_config
        if sc is not None and sc.enable_sequence_parallelism and sc.sequence_parallel_size > 1:
            if sc.sequence_parallelism_mode not in self.supported_sp_modes:
                raise ValueError(f"{type(self).__name__} does not support sequence parallelism mode {sc.sequence_parallelism_mode}")

    def get_held_layers(self) -> list[str]:
        sm = self.shard_config.pipeline_stage_manager if self.shard_config is not None else None
        if sm is None:
            return self.get_all_modules(self.model.config)
        return sm.held_module_names()

    def split_sizes(self, path: str, module) -> list[int] | None:
        return None

    def get_shared_params(self) -> list[dict]:
        return []
