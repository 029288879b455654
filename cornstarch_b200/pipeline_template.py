"""``PipelineTemplate``: which named modules of a model live on which pipeline stage.

Same contract as the reference class (cornstarch/pipeline_template.py:10-134): a template is
``(model_name, modules_per_stage)`` plus planner hints (``latency``, ``kstar_latency``,
``mem_required``); ``get_modules(model)`` returns the model's ordered pipeline units, which for a
:class:`ModalModuleBase` are the encoder's units prefixed with ``module.`` followed by the projector's
prefixed with ``projector.``.  Here the names come from each model class's ``module_names(config)``
instead of from a per-model policy class.
"""

from __future__ import annotations

import re
from typing import Optional

from torch import nn


def _fullname(obj) -> str:
    klass = obj.__class__
    module = klass.__module__
    if module == "builtins":
        return klass.__qualname__
    return module + "." + klass.__qualname__


class PipelineTemplate:
    """A template for a single pipeline that can be used to instantiate identical pipelines."""

    @staticmethod
    def get_model_name(model: nn.Module) -> str:
        return _fullname(model)

    @staticmethod
    def get_modules(model: nn.Module) -> list[str]:
        from .multimodal.modeling import ModalModuleBase
        from .shardformer.policies.auto_policy import policy_for_model

        if isinstance(model, ModalModuleBase):
            names = [f"module.{m}" for m in type(policy_for_model(model.module)).get_all_modules(model.module.config)]
            if model.projector is not None:
                names += [f"projector.{m}" for m in type(policy_for_model(model.projector)).get_all_modules(model.projector.config)]
            return names
        return type(policy_for_model(model)).get_all_modules(model.config)

    @staticmethod
    def find_pipeline_template(pipeline_templates: list["PipelineTemplate"], num_stages: int) -> Optional["PipelineTemplate"]:
        return next((t for t in pipeline_templates if t.num_stages == num_stages), None)

    def __init__(self, model_name: str, modules_per_stage: list[list[str]], latency: float = 0.0,
                 kstar_latency: float = 0.0, mem_required: int = 0):
        self.model_name = model_name
        self.modules_per_stage = modules_per_stage
        self.pseudo_latency = latency  # latency measured with 4 * num_stages micro-batches
        self.kstar_latency = kstar_latency
        self.mem_required = mem_required

    def __repr__(self) -> str:
        return f"PipelineTemplate({self.model_name}, {self.num_stages} stages)"

    def latency(self, num_microbatches: int) -> float:
        """Estimated latency with the actual number of micro-batches."""
        assert num_microbatches >= self.num_stages, "Number of microbatches must be >= num_stages."
        return self.pseudo_latency + self.kstar_latency * (num_microbatches - 4 * self.num_stages)

    def get_num_layers_per_stage(self) -> list[int]:
        """Per stage, the number of module names that contain ``.<digit>`` (repeated transformer layers)."""
        return [sum(bool(re.search(r"\.\d", s)) for s in modules) for modules in self.modules_per_stage]

    @property
    def num_layers(self) -> int:
        return sum(len(stage) for stage in self.modules_per_stage)

    @property
    def num_stages(self) -> int:
        return len(self.modules_per_stage)

    def __eq__(self, other) -> bool:
        return isinstance(other, PipelineTemplate) and self.model_name == other.model_name and hash(self) == hash(other)

    def __hash__(self) -> int:
        return hash(tuple(tuple(m) for m in self.modules_per_stage))

    @staticmethod
    def even_split(model: nn.Module, num_stages: int) -> "PipelineTemplate":
        """Convenience: first/last units stay with the first/last stage, repeated layers are split evenly."""
        names = PipelineTemplate.get_modules(model)
        layer_idx = [i for i, n in enumerate(names) if re.search(r"\.\d", n)]
        assert len(layer_idx) >= num_stages, "more stages than layers"
        first, last = layer_idx[0], layer_idx[-1]
        n_layers = len(layer_idx)
        per = [n_layers // num_stages + (1 if s < n_layers % num_stages else 0) for s in range(num_stages)]
        stages, cur = [], first
        for s in range(num_stages):
            chunk = names[cur : cur + per[s]]
            cur += per[s]
            if s == 0:
                chunk = names[:first] + chunk
            if s == num_stages - 1:
                chunk = chunk + names[last + 1 :]
            stages.append(chunk)
        return PipelineTemplate(PipelineTemplate.get_model_name(model), stages)
