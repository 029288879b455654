"""``ModalParallelPlugin``: the parallel plan of ONE modality (an encoder or the language model).

Constructor arguments follow the reference (cornstarch/plugin/multimodal_parallel_plugin/
modal_parallel_plugin.py:72-101): ``tp_size``, ``sp_size``, ``sequence_parallelism_mode``
(``"ring_attn"`` = context parallelism, ``"all_to_all"`` = Ulysses), ``pipeline_template``,
``context_parallel_distribution_mode``, ``custom_policy``.  ``configure`` shards the modality's module(s)
with :class:`ShardFormer`.
"""

from __future__ import annotations

from typing import Optional

import torch.nn as nn

from ..multimodal.modeling import ModalModuleBase
from ..pipeline_template import PipelineTemplate
from ..shardformer.policies.auto_policy import policy_for_model
from ..shardformer.shard.shard_config import ContextParallelDistributionMode, ShardConfig
from ..shardformer.shard.shardformer import ShardFormer


class ModalParallelPlugin:
    def __init__(self, tp_size: int = 1, sp_size: int = 1, sequence_parallelism_mode: Optional[str] = None,
                 pipeline_template: Optional[PipelineTemplate] = None,
                 context_parallel_distribution_mode: ContextParallelDistributionMode | str = ContextParallelDistributionMode.MAKESPAN_MIN,
                 cpu_offload: bool = False, custom_policy=None, ep_size: int = 1,
                 ep_capacity_factor: Optional[float] = None, ep_capacity_tokens: Optional[int] = None):
        if sp_size > 1:
            assert sequence_parallelism_mode in ("ring_attn", "all_to_all"), (
                "sequence_parallelism_mode must be 'ring_attn' or 'all_to_all' when sp_size > 1")
        self.tp_size = tp_size
        self.sp_size = sp_size
        # expert parallelism (MoE language models): the experts of every sparse block are sharded over the data-parallel
        # ranks of the stage that holds the block, so ep_size must equal the data-parallel degree.  With a capacity factor
        # the dispatch has static shapes and makes no host read (parallel/ep.py).
        self.ep_size = ep_size
        self.ep_capacity_factor = ep_capacity_factor
        self.ep_capacity_tokens = ep_capacity_tokens  # fixed token count that sizes the exchange (ranks with unequal batches)
        self.sequence_parallelism_mode = sequence_parallelism_mode if sp_size > 1 else None
        self.pipeline_template = pipeline_template
        self.context_parallel_distribution_mode = (
            ContextParallelDistributionMode(context_parallel_distribution_mode)
            if isinstance(context_parallel_distribution_mode, str) else context_parallel_distribution_mode)
        self.cpu_offload = cpu_offload
        self.custom_policy = custom_policy
        self.shard_config: ShardConfig | None = None

    def make_shard_config(self, tp_group, sp_group, stage_manager, device=None, dtype=None, ep_group=None, **flags) -> ShardConfig:
        self.shard_config = ShardConfig(
            tensor_parallel_process_group=tp_group,
            sequence_parallel_process_group=sp_group,
            pipeline_stage_manager=stage_manager,
            pipeline_template=self.pipeline_template,
            enable_tensor_parallelism=self.tp_size > 1,
            enable_sequence_parallelism=self.sp_size > 1,
            sequence_parallelism_mode=self.sequence_parallelism_mode,
            context_parallel_distribution_mode=self.context_parallel_distribution_mode,
            expert_parallel_process_group=ep_group,
            extra_kwargs={"device": device, "dtype": dtype},
            **flags,
        )
        return self.shard_config

    def configure(self, model: nn.Module, shard_config: ShardConfig | None = None, stage_manager=None):
        """Shard ``model`` (a ``ModalModuleBase`` or a language model) in place and return it."""
        sc = shard_config or self.shard_config
        assert sc is not None, "call make_shard_config first"
        former = ShardFormer(sc)
        if isinstance(model, ModalModuleBase):
            held = stage_manager.held_module_names() if stage_manager is not None else None
            self._configure_modal_module(model, sc, former, held)
        else:
            former.optimize(model, self.custom_policy or policy_for_model(model))
        return model

    def _configure_modal_module(self, modal: ModalModuleBase, sc: ShardConfig, former: ShardFormer, held: list[str] | None):
        """Encoder units are named ``module.<unit>``; the projector's ``projector.<unit>`` (last stage only)."""
        from ..shardformer.policies.multimodal import ModalModulePolicy

        pol = ModalModulePolicy()
        pol.set_model(modal)
        pol.set_shard_config(sc)
        pol.shard(sc, held)


from ..shardformer.policies.multimodal import _FixedHeld  # noqa: E402,F401  (used by the colocated plugin)
