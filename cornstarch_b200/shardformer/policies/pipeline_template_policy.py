"""Base class of every policy: the ordered pipeline units of a model and the template sanity check
(cornstarch/shardformer/policies/pipeline_template_policy.py:8-35 in the reference)."""

from __future__ import annotations

import itertools
from abc import ABC, abstractmethod


class PipelineTemplatePolicyBase(ABC):
    skip_replaced_modules: bool = True

    @staticmethod
    @abstractmethod
    def get_all_modules(config) -> list[str]:
        """Ordered names of the modules that can be assigned to pipeline stages."""

    @abstractmethod
    def pipeline_template_sanity_check(self, template) -> None:
        """Raise ``ValueError`` when ``template`` cannot be used with this model."""


def check_template_covers(template, modules: list[str], first: list[str], last: list[str], model_name: str | None = None):
    """Shared sanity check: exact flattened module list, first-stage and last-stage constraints."""
    flat = list(itertools.chain(*template.modules_per_stage))
    if flat != modules:
        raise ValueError(f"Modules in the pipeline template do not match the modules in the model: {flat} vs {modules}.")
    for name in first:
        if name in modules and name not in template.modules_per_stage[0]:
            raise ValueError(f"The module {name} must be in the first stage.")
    for name in last:
        if name in modules and name not in template.modules_per_stage[-1]:
            raise ValueError(f"The module {name} must be in the last stage.")
    for stage in template.modules_per_stage:
        if not stage:
            raise ValueError("A pipeline stage holds no module.")
