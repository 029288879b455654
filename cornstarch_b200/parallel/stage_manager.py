"""Pipeline stage manager for a DAG of modalities: encoder branches feed the LLM's first stage.

For the rank at hand it answers: which modality am I, which stage inside it, who are my previous and next
ranks.  Encoder last stages send to the LLM's first stage (same dp/sp/tp coordinates); the LLM's last
stage wraps around to the encoders' first stages, as in the reference
(cornstarch/plugin/multimodal_parallel_plugin/multimodal_stage_manager.py:22-372; expected tables in
tests/test_plugins/multimodal_parallel_plugin/test_multimodal_stage_manager.py:31-110 of the reference).
Pure index math on the mesh: no process group is needed to construct it.
"""

from __future__ import annotations

import itertools


from ..pipeline_template import PipelineTemplate
from .mesh import MultiModalProcessGroupMesh


class MultiModalPipelineStageManager:
    def __init__(self, pg_mesh: MultiModalProcessGroupMesh, pipeline_axis: int = 0):
        self.pg_mesh = pg_mesh
        self.pipeline_axis = pipeline_axis
        self.is_interleave = False
        self.num_model_chunks = 1
        self.stage_index_to_modal: list[PipelineTemplate] = list(itertools.chain.from_iterable(
            [modal] * modal.num_stages for modal in pg_mesh.topological_sorted_modals))
        coords = pg_mesh.coords
        ax = pipeline_axis
        self.my_modal = self.stage_index_to_modal[coords[0][ax]]
        enc = list(pg_mesh.encoder_templates.keys())
        llm = pg_mesh.llm_template[0] if pg_mesh.llm_template is not None else None
        if self.my_modal in enc:
            prev_modals = [llm] if llm is not None else []
            next_modals = [llm] if llm is not None else []
        else:
            prev_modals, next_modals = list(enc), list(enc)

        def first_stage_of(m):
            return self.stage_index_to_modal.index(m)

        def last_stage_of(m):
            return len(self.stage_index_to_modal) - 1 - self.stage_index_to_modal[::-1].index(m)

        prev_coords, next_coords = [], []
        n_stages_total = pg_mesh.shape[ax]
        for c in coords:
            s = c[ax]
            if s == 0 or self.stage_index_to_modal[s - 1] != self.my_modal:
                for m in prev_modals:
                    prev_coords.append(c[:ax] + (last_stage_of(m),) + c[ax + 1 :])
            else:
                prev_coords.append(c[:ax] + (s - 1,) + c[ax + 1 :])
            if s == n_stages_total - 1 or self.stage_index_to_modal[s + 1] != self.my_modal:
                for m in next_modals:
                    next_coords.append(c[:ax] + (first_stage_of(m),) + c[ax + 1 :])
            else:
                next_coords.append(c[:ax] + (s + 1,) + c[ax + 1 :])
        self.prev_ranks: list[int] = sorted({int(pg_mesh.mesh[c]) for c in prev_coords})
        self.next_ranks: list[int] = sorted({int(pg_mesh.mesh[c]) for c in next_coords})

    # ------------------------------------------------------------------ roles
    def _modal_stage_range(self, modal) -> tuple[int, int]:
        first = self.stage_index_to_modal.index(modal)
        return first, first + modal.num_stages

    def is_first_stage(self, ignore_chunk: bool = False, check_only_in_modal: bool = True) -> bool:
        """First stage of my modality; with ``check_only_in_modal=False``: first stage of an encoder (or of the LLM when there are no encoders)."""
        if self.stage_in_modal != 0:
            return False
        if check_only_in_modal:
            return True
        if len(self.pg_mesh.encoder_templates) > 0:
            return self.my_modal in self.pg_mesh.encoder_templates
        return True

    def is_last_stage(self, ignore_chunk: bool = False, check_only_in_modal: bool = True) -> bool:
        """Last stage of my modality; with ``check_only_in_modal=False``: last stage of the LLM (or of an encoder when there is no LLM)."""
        if self.stage_in_modal != self.my_modal.num_stages - 1:
            return False
        if check_only_in_modal:
            return True
        if self.pg_mesh.llm_template is not None:
            return self.my_modal == self.pg_mesh.llm_template[0]
        return True

    def get_prev_rank(self) -> int:
        assert len(self.prev_ranks) == 1
        return self.prev_ranks[0]

    def get_next_rank(self) -> int:
        assert len(self.next_ranks) == 1
        return self.next_ranks[0]

    def get_prev_ranks(self) -> list[int]:
        return self.prev_ranks

    def get_next_ranks(self) -> list[int]:
        return self.next_ranks

    @property
    def num_stages(self) -> int:
        return self.pg_mesh.size(self.pipeline_axis)

    @property
    def num_stages_in_modal(self) -> int:
        return self.my_modal.num_stages

    @property
    def stage(self) -> int:
        return self.pg_mesh.coords[0][self.pipeline_axis]

    @property
    def stage_in_modal(self) -> int:
        return self.stage - self.stage_index_to_modal.index(self.my_modal)

    @property
    def is_encoder(self) -> bool:
        return self.my_modal in self.pg_mesh.encoder_templates

    # ------------------------------------------------------------------ layer distribution
    def distribute_layers(self, num_layers: int | None = None, num_stages: int | None = None, num_model_chunks: int | None = None) -> list[int]:
        """Number of repeated layers on every stage of the whole DAG (concatenated over modalities)."""
        return list(itertools.chain.from_iterable(m.get_num_layers_per_stage() for m in self.pg_mesh.topological_sorted_modals))

    def get_stage_index(self, layers_per_stage: list[int], stage: int | None = None, num_model_chunks=None, num_stages=None) -> tuple[int, int]:
        """Modal-relative ``[start, end)`` layer range of ``stage`` (default: mine); ``(0, 0)`` if that stage is another modality's."""
        stage = self.stage if stage is None else stage
        modal = self.stage_index_to_modal[stage]
        if modal != self.my_modal:
            return (0, 0)
        first, _ = self._modal_stage_range(modal)
        start = sum(layers_per_stage[first:stage])
        return (start, start + layers_per_stage[stage])

    def held_module_names(self) -> list[str]:
        """Names of the pipeline units of my modality that my stage owns."""
        return list(self.my_modal.modules_per_stage[self.stage_in_modal])
