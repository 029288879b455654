"""Policy of the modality wrappers (``ModalEncoderModule`` / ``ModalDecoderModule``): an encoder (or decoder) module plus
its projector, sharded by the policies of the two parts.

Pipeline units of a wrapper are named ``module.<unit>`` for the wrapped model's own units and ``projector.<unit>`` for
the projector, which lives on the wrapper's last stage only.  Corresponds to ``ModalModulePolicy`` of the reference
(cornstarch/shardformer/policies/multimodal.py:139-234), which merges the ``module_policy()`` dictionaries and held
layers of the wrapped model's policy and the projector's policy.
"""

from __future__ import annotations

import copy

from .base_policy import ModelPolicy


class _FixedHeld:
    """Minimal stage-manager stand-in that reports a fixed list of held units."""

    def __init__(self, names):
        self._names = list(names)

    def held_module_names(self):
        return self._names


class ModalModulePolicy(ModelPolicy):
    """Units, held layers and sharding of a modality wrapper, delegated to the policies of its parts."""

    is_modal_module_policy = True

    def _parts(self):
        from .auto_policy import policy_for_model

        inner = policy_for_model(self.model.module)
        proj = policy_for_model(self.model.projector) if getattr(self.model, "projector", None) is not None else None
        return inner, proj

    @classmethod
    def get_all_modules(cls, config) -> list[str]:
        raise NotImplementedError("a modality wrapper has no configuration of its own: use all_modules() on a bound policy")

    def all_modules(self) -> list[str]:
        inner, proj = self._parts()
        names = [f"module.{n}" for n in type(inner).get_all_modules(self.model.module.config)]
        if proj is not None:
            names += [f"projector.{n}" for n in type(proj).get_all_modules(self.model.projector.config)]
        return names

    def pipeline_template_sanity_check(self, template) -> None:
        import itertools

        flat = list(itertools.chain(*template.modules_per_stage))
        want = self.all_modules()
        if flat != want:
            raise ValueError(f"Modules in the pipeline template do not match the modules in the model: {flat} vs {want}.")
        for n in flat:
            if n.startswith("projector.") and n not in template.modules_per_stage[-1]:
                raise ValueError("The projector must be in the last stage.")

    def get_held_layers(self) -> list[str]:
        sm = self.shard_config.pipeline_stage_manager if self.shard_config is not None else None
        return self.all_modules() if sm is None else sm.held_module_names()

    def shard(self, shard_config, held: list[str] | None = None):
        """Shard the wrapped model and the projector in place with their own policies."""
        from ..shard.shardformer import ShardFormer
        from .auto_policy import policy_for_model

        modal, sc = self.model, shard_config
        if held is None and sc.pipeline_stage_manager is not None:
            held = sc.pipeline_stage_manager.held_module_names()
        enc_held = None if held is None else [h[len("module."):] for h in held if h.startswith("module.")]
        proj_held = None if held is None else [h for h in held if h.startswith("projector.")]
        enc_sc = copy.copy(sc)
        if enc_held is not None:
            enc_sc.pipeline_stage_manager = _FixedHeld(enc_held)
            enc_sc.pipeline_template = None
        ShardFormer(enc_sc).optimize(modal.module, policy_for_model(modal.module))
        if modal.projector is not None:
            if proj_held is not None and not proj_held:
                modal.projector = None  # the projector lives on the wrapper's last stage only
            else:
                proj_sc = copy.copy(sc)
                proj_sc.pipeline_stage_manager = None
                proj_sc.pipeline_template = None
                proj_sc.enable_sequence_parallelism = False
                proj_sc.sequence_parallelism_mode = None
                ShardFormer(proj_sc).optimize(modal.projector, policy_for_model(modal.projector))
                if sc.enable_sequence_parallelism and sc.sequence_parallel_size > 1:
                    from ...parallel.comm import gather_forward_split_backward

                    sp_group, sp = sc.sequence_parallel_process_group, sc.sequence_parallel_size
                    modal.projector.post_projection = lambda x: gather_forward_split_backward(x, 1, sp_group, float(sp))
        return modal
