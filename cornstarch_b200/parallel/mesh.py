"""Process-group mesh for modality-parallel training: a 4-D grid ``(pp, dp, sp, tp)`` of ranks.

The grid is built stage by stage: every modality (encoders in dict order, then the LLM) contributes
``num_stages`` rows; inside a stage, for each data-parallel replica and each sequence-parallel index,
``tp`` fresh ranks are allocated and *repeated* to fill the widest tp / sp of any modality.  A rank can
therefore sit at several coordinates.  The data-parallel degree is inferred:
``world_size // sum(stages * tp * sp)``.  This reproduces the layout of the reference
(cornstarch/plugin/multimodal_parallel_plugin/modal_process_group_mesh.py:38-142; expected meshes in
tests/test_plugins/multimodal_parallel_plugin/test_modal_process_group_mesh.py:28-358 of the reference).

Everything here is index arithmetic on a numpy array and needs no initialised process group, so a
single process can compute the view of every rank (used by the tests for world sizes up to 132).
``torch.distributed`` groups are created lazily and collectively by :meth:`get_group_along_axis`.
An optional expert-parallel view (``ep``) re-uses the data-parallel axis.
"""

from __future__ import annotations

import itertools
from typing import Optional

import numpy as np
import torch.distributed as dist

from ..pipeline_template import PipelineTemplate


class MultiModalProcessGroupMesh:
    pp_axis, dp_axis, sp_axis, tp_axis = 0, 1, 2, 3

    def __init__(self, encoder_templates: Optional[dict[PipelineTemplate, int | tuple[int, int]]] = None,
                 llm_template: Optional[tuple[PipelineTemplate, int, int]] = None,
                 world_size: int | None = None, rank: int | None = None):
        encoder_templates = dict(encoder_templates or {})
        for tpl, sizes in list(encoder_templates.items()):
            if isinstance(sizes, int):
                encoder_templates[tpl] = (sizes, 1)
        if world_size is None:
            assert dist.is_initialized(), "Please initialize torch.distributed first (or pass world_size and rank)."
            world_size, rank = dist.get_world_size(), dist.get_rank()
        self._world_size, self._rank = world_size, rank
        self.encoder_templates = encoder_templates
        self.llm_template = llm_template
        self.decoder_templates: dict = {}
        self.topological_sorted_modals: list[PipelineTemplate] = [*encoder_templates.keys(), *([] if llm_template is None else [llm_template[0]])]

        sizes = {tpl: ts for tpl, ts in encoder_templates.items()}
        if llm_template is not None:
            sizes[llm_template[0]] = (llm_template[1], llm_template[2])
        ranks_per_replica = sum(tpl.num_stages * tp * sp for tpl, (tp, sp) in sizes.items())
        assert world_size % ranks_per_replica == 0, (
            f"The world size {world_size} must be divisible by num_ranks per replica {ranks_per_replica}.")
        dp_size = world_size // ranks_per_replica
        max_tp = max(tp for tp, _ in sizes.values())
        max_sp = max(sp for _, sp in sizes.values())
        for tp, sp in sizes.values():
            assert max_tp % tp == 0, f"tp size {tp} must divide the largest tp size {max_tp}"
            assert max_sp % sp == 0, f"sp size {sp} must divide the largest sp size {max_sp}"

        self.modal_to_ranks: dict[PipelineTemplate, list[int]] = {}
        rows = []
        nxt = 0
        for modal in self.topological_sorted_modals:
            tp, sp = sizes[modal]
            first = nxt
            for _stage in range(modal.num_stages):
                stage_rows = []
                for _d in range(dp_size):
                    replica = []
                    for _s in range(sp):
                        row = [r for r in range(nxt, nxt + tp) for _ in range(max_tp // tp)]
                        nxt += tp
                        replica.extend([row] * (max_sp // sp))
                    stage_rows.append(replica)
                rows.append(stage_rows)
            self.modal_to_ranks[modal] = list(range(first, nxt))
        self._mesh = np.array(rows, dtype=np.int64)
        self._shape = self._mesh.shape
        self._sizes = sizes
        self._coords = self.unravel(rank, self._mesh) if rank is not None else []
        self._groups: dict[tuple[int, ...], dist.ProcessGroup] = {}

    # ------------------------------------------------------------------ index math
    @property
    def shape(self) -> tuple[int, ...]:
        return self._shape

    @property
    def rank(self) -> int:
        return self._rank

    @property
    def coords(self) -> list[tuple[int, ...]]:
        return self._coords

    @property
    def mesh(self) -> np.ndarray:
        return self._mesh

    def size(self, axis: int) -> int:
        return self._shape[axis]

    @property
    def dp_size(self) -> int:
        return self._shape[self.dp_axis]

    @staticmethod
    def unravel(rank: int, mesh: np.ndarray) -> list[tuple[int, ...]]:
        """All coordinates at which ``rank`` appears."""
        return [tuple(int(i) for i in c) for c in zip(*np.where(mesh == rank))]

    def modal_of_rank(self, rank: int | None = None) -> PipelineTemplate:
        rank = self._rank if rank is None else rank
        for modal, ranks in self.modal_to_ranks.items():
            if rank in ranks:
                return modal
        raise ValueError(f"rank {rank} is not in the mesh")

    def parallel_sizes(self, modal: PipelineTemplate) -> tuple[int, int]:
        return self._sizes[modal]

    def rank_sets_along_axis(self, axis: int | list[int]) -> list[tuple[int, ...]]:
        """Distinct sorted rank tuples obtained by varying ``axis`` with all other coordinates fixed (deterministic order)."""
        axes = [axis] if isinstance(axis, int) else list(axis)
        reduced = [1 if a in axes else s for a, s in enumerate(self._shape)]
        seen, out = set(), []
        for base in itertools.product(*[range(s) for s in reduced]):
            idx = tuple(slice(None) if a in axes else base[a] for a in range(len(self._shape)))
            ranks = tuple(sorted(set(int(r) for r in np.asarray(self._mesh[idx]).reshape(-1))))
            if ranks not in seen:
                seen.add(ranks)
                out.append(ranks)
        return out

    def my_rank_sets_along_axis(self, axis: int | list[int], rank: int | None = None) -> list[tuple[int, ...]]:
        rank = self._rank if rank is None else rank
        return [rs for rs in self.rank_sets_along_axis(axis) if rank in rs]

    def get_ranks_in_group(self, group) -> list[int]:
        for ranks, g in self._groups.items():
            if g is group:
                return list(ranks)
        return dist.get_process_group_ranks(group)

    # ------------------------------------------------------------------ torch.distributed groups
    def _get_group(self, ranks: tuple[int, ...], backend: str | None = None):
        if ranks not in self._groups:
            self._groups[ranks] = dist.new_group(list(ranks), backend=backend)
        return self._groups[ranks]

    def get_group_along_axis(self, axis: int | list[int], indices_at_axis=None, backend: str | None = None):
        """Create (collectively, on every rank, in the same order) all groups along ``axis``; return mine.

        A list is returned for the pipeline axis (a rank of a narrow modality belongs to several pipelines),
        a single group otherwise.
        """
        axes = [axis] if isinstance(axis, int) else list(axis)
        if self.pp_axis in axes:
            assert len(axes) == 1, "Only one axis is allowed for pp group."
        mine = []
        for ranks in self.rank_sets_along_axis(axes):
            g = self._get_group(ranks, backend)
            if self._rank in ranks:
                mine.append(g)
        if len(mine) > 1 or axes[0] == self.pp_axis:
            return mine
        return mine[0]

    def create_group(self, ranks: list[int], backend: str | None = None):
        return self._get_group(tuple(sorted(ranks)), backend)
