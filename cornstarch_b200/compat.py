"""Import-path compatibility with the reference package.

``import cornstarch_b200.compat`` (or ``cornstarch_b200.compat.install()``) registers aliases in
``sys.modules`` so that user scripts written against the reference keep their imports::

    from cornstarch.models.multimodal_language_model import MultimodalModel, ModalEncoderModule, MultimodalProjector
    from cornstarch.pipeline_template import PipelineTemplate
    from cornstarch.plugin.multimodal_parallel_plugin import ModalParallelPlugin, MultimodalParallelPlugin
    from cornstarch.shardformer.shard.shard_config import ShardConfig, ContextParallelDistributionMode
    from cornstarch.kernel.interface import create_bitfield_attention_mask
    from colossalai.booster import Booster

Nothing is aliased when a real ``cornstarch`` package is already imported.
"""

from __future__ import annotations

import importlib
import sys
import types

_ALIASES = {
    "cornstarch": "cornstarch_b200",
    "cornstarch.pipeline_template": "cornstarch_b200.pipeline_template",
    "cornstarch.models": "cornstarch_b200.models",
    "cornstarch.models.multimodal_language_model": "cornstarch_b200.multimodal",
    **{f"cornstarch.models.multimodal_language_model.{m}": "cornstarch_b200.multimodal"
       for m in ("modeling_multimodal_language_model", "processing_multimodal_language_model",
                 "configuration_multimodal_language_model")},
    **{f"cornstarch.models.{m}": "cornstarch_b200.models.evaclip"
       for m in ("evaclip", "evaclip.modeling_evaclip", "evaclip.configuration_evaclip")},
    **{f"cornstarch.models.{m}": "cornstarch_b200.models.vision_extra"
       for m in ("intern_vit", "intern_vit.modeling_intern_vit", "intern_vit.configuration_intern_vit")},
    "cornstarch.kernel": "cornstarch_b200.kernel",
    "cornstarch.kernel.interface": "cornstarch_b200.kernel.interface",
    "cornstarch.kernel.bitfield_attention": "cornstarch_b200.kernel.bitfield_attention",
    "cornstarch.kernel.attention": "cornstarch_b200.kernel.attention",
    "cornstarch.models.intern_vit.flash_attention": "cornstarch_b200.kernel.attention",  # FlashAttention module
    "cornstarch.plugin": "cornstarch_b200.plugin",
    "cornstarch.plugin.multimodal_parallel_plugin": "cornstarch_b200.plugin.multimodal_parallel_plugin",
    # the sub-modules of that package: every one resolves to the module that exports all of the package's names
    "cornstarch.plugin.multimodal_parallel_plugin.modal_parallel_plugin": "cornstarch_b200.plugin.modal_parallel_plugin",
    "cornstarch.plugin.multimodal_parallel_plugin.multimodal_parallel_plugin": "cornstarch_b200.plugin.multimodal_parallel_plugin",
    "cornstarch.plugin.multimodal_parallel_plugin.modal_process_group_mesh": "cornstarch_b200.parallel.mesh",
    "cornstarch.plugin.multimodal_parallel_plugin.multimodal_stage_manager": "cornstarch_b200.parallel.stage_manager",
    "cornstarch.plugin.multimodal_parallel_plugin.multimodal_1f1b": "cornstarch_b200.parallel.schedule",
    "cornstarch.plugin.multimodal_parallel_plugin.multimodal_parallel_checkpoint_io": "cornstarch_b200.plugin.checkpoint_io",
    "cornstarch.plugin.encoders_colocated_plugin": "cornstarch_b200.plugin.encoders_colocated_plugin",
    "cornstarch.plugin.encoders_colocated_plugin.encoders_colocated_plugin": "cornstarch_b200.plugin.encoders_colocated_plugin",
    "cornstarch.plugin.heterogeneous_parallel_plugin": "cornstarch_b200.plugin.heterogeneous_parallel_plugin",
    **{f"cornstarch.plugin.heterogeneous_parallel_plugin.{m}": "cornstarch_b200.plugin.heterogeneous_parallel_plugin"
       for m in ("heterogeneous_dataloader", "heterogeneous_parallel_module", "heterogeneous_parallel_plugin",
                 "heterogeneous_process_group_mesh", "heterogeneous_stage_manager")},
    **{f"cornstarch.plugin.encoders_colocated_plugin.{m}": "cornstarch_b200.plugin.encoders_colocated_plugin"
       for m in ("encoders_colocated_stage_manager", "process_group_mesh")},
    "cornstarch.shardformer": "cornstarch_b200.shardformer",
    "cornstarch.shardformer.shard": "cornstarch_b200.shardformer.shard",
    "cornstarch.shardformer.shard.shard_config": "cornstarch_b200.shardformer.shard.shard_config",
    "cornstarch.shardformer.shard.shardformer": "cornstarch_b200.shardformer.shard.shardformer",
    "cornstarch.shardformer.policies": "cornstarch_b200.shardformer.policies",
    "cornstarch.shardformer.policies.auto_policy": "cornstarch_b200.shardformer.policies.auto_policy",
    "cornstarch.shardformer.policies.pipeline_template_policy": "cornstarch_b200.shardformer.policies.pipeline_template_policy",
    "cornstarch.shardformer.policies.multimodal": "cornstarch_b200.shardformer.policies.multimodal",
    **{f"cornstarch.shardformer.policies.{m}": "cornstarch_b200.shardformer.policies.models"
       for m in ("bert", "clip", "dinov2", "evaclip", "gemma", "gemma2", "gemma3", "gpt2", "intern_vit", "llama", "llama4",
                 "mistral", "mixtral", "opt", "phi3", "phi4_multimodal", "pixtral", "qwen2", "qwen2_audio", "qwen2_vision",
                 "qwen3", "qwen3_moe", "siglip", "vit", "whisper")},
    "cornstarch.shardformer.layers": "cornstarch_b200.shardformer.layers",
    "cornstarch.shardformer.layers.utils": "cornstarch_b200.parallel.cp",
    "cornstarch.shardformer.layers.operation": "cornstarch_b200.parallel.comm",
    "cornstarch.shardformer.layers.context_parallel_bitfield_attention": "cornstarch_b200.shardformer.layers.context_parallel_bitfield_attention",
    "cornstarch.shardformer.layers.context_parallel_attention": "cornstarch_b200.shardformer.layers.context_parallel_attention",
    "cornstarch.testing": "cornstarch_b200.testing",
    "cornstarch.testing.timer": "cornstarch_b200.testing.timer",
    "cornstarch.testing.dcgm": "cornstarch_b200.testing.dcgm",
}


def install(force: bool = False) -> None:
    if "cornstarch" in sys.modules and not force and getattr(sys.modules["cornstarch"], "__name__", "") != "cornstarch_b200":
        return
    for alias, target in _ALIASES.items():
        try:
            sys.modules[alias] = importlib.import_module(target)
        except ImportError:
            continue
    if "colossalai" not in sys.modules:
        col = types.ModuleType("colossalai")
        booster = types.ModuleType("colossalai.booster")
        from .booster import Booster

        booster.Booster = Booster
        col.booster = booster
        sys.modules["colossalai"] = col
        sys.modules["colossalai.booster"] = booster


install()
