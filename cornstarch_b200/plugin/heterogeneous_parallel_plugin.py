"""Heterogeneous pipelines (Oobleck style): the data-parallel replicas of ONE model are pipelines with
different numbers of stages, built from a set of :class:`PipelineTemplate`s.

* :class:`HeterogeneousProcessGroupMesh` is a ``[pipeline][pipeline unit][tp]`` table of ranks: unit ``u`` of
  pipeline ``p`` is held by the ranks of the stage that owns it, so the data-parallel group of a unit is the
  set of ranks that hold it across pipelines (one group per unit, per tp index).
* Gradients are reduced per unit over that group.  Pipelines run different numbers of micro-batches per
  step, so each pipeline weights its loss by ``its micro-batches / all micro-batches`` and the reduction is
  a SUM: the result is the exact mean over the global batch.
* :class:`HeterogeneousDataLoader` / :class:`HeterogeneousBatchSampler` give pipeline ``i``
  ``microbatch_size * num_microbatches[i]`` samples of every global batch.
* ``configure(..., forced=True)`` re-wraps an already wrapped model after ``set_pipelines`` was called
  again (re-planning after a membership change); released layers are re-created from their placeholders.

Public names and call sequence follow the reference
(cornstarch/plugin/heterogeneous_parallel_plugin/: heterogeneous_parallel_plugin.py:53-366,
heterogeneous_process_group_mesh.py:66-109, heterogeneous_stage_manager.py:13-130,
heterogeneous_dataloader.py:12-180, heterogeneous_parallel_module.py:20-109).
"""

from __future__ import annotations

import math
from typing import Callable, Iterator, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import BatchSampler, DataLoader, Dataset

from ..optim.fused_adamw import FusedAdamW, split_decay_groups
from ..optim.wrapper import OptimizerWrapper
from ..parallel.schedule import MultimodalEncoderTrainingOneForwardOneBackwardSchedule
from ..pipeline_template import PipelineTemplate
from ..shardformer.policies.auto_policy import policy_for_model
from ..shardformer.shard.shard_config import ShardConfig
from ..shardformer.shard.shardformer import ShardFormer
from .multimodal_parallel_plugin import PRECISION


class HeterogeneousProcessGroupMesh:
    dp_axis, pp_axis, tp_axis = 0, 1, 2

    def __init__(self, pipelines: list[PipelineTemplate], tp_size: int, ranks: Optional[list[int]] = None,
                 rank: int | None = None):
        assert pipelines, "At least one pipeline template must be given."
        assert all(p.num_layers == pipelines[0].num_layers for p in pipelines), (
            "All pipeline templates must have the same number of layers.")
        self.pipelines = pipelines
        self._shape = (len(pipelines), pipelines[0].num_layers, tp_size)
        self._rank = dist.get_rank() if rank is None else rank
        n = tp_size * sum(p.num_stages for p in pipelines)
        ranks = list(range(n)) if ranks is None else ranks
        mesh = np.empty(self._shape, dtype=np.int64)
        nxt = 0
        for pi, p in enumerate(pipelines):
            unit = 0
            for modules in p.modules_per_stage:
                stage_ranks = ranks[nxt : nxt + tp_size]
                for _ in modules:
                    mesh[pi, unit] = stage_ranks
                    unit += 1
                nxt += tp_size
        self._mesh = mesh
        self._coords = [tuple(int(i) for i in c) for c in zip(*np.where(mesh == self._rank))]
        self._groups: dict[tuple[int, ...], dist.ProcessGroup] = {}

    @property
    def shape(self):
        return self._shape

    @property
    def mesh(self):
        return self._mesh

    @property
    def coords(self):
        return self._coords

    @property
    def rank(self):
        return self._rank

    def size(self, axis: int) -> int:
        return self._shape[axis]

    def rank_sets_along_axis(self, axis: int) -> list[tuple[int, ...]]:
        out, seen = [], set()
        other = [a for a in range(3) if a != axis]
        for i in range(self._shape[other[0]]):
            for j in range(self._shape[other[1]]):
                idx = [slice(None)] * 3
                idx[other[0]], idx[other[1]] = i, j
                rs = tuple(sorted(set(int(r) for r in self._mesh[tuple(idx)].reshape(-1))))
                if rs not in seen:
                    seen.add(rs)
                    out.append(rs)
        return out

    def get_group_along_axis(self, axis: int, backend: str | None = None):
        """All groups along ``axis`` are created collectively; returns mine (a list for the dp axis: one per held unit)."""
        mine = []
        for rs in self.rank_sets_along_axis(axis):
            if rs not in self._groups:
                self._groups[rs] = dist.new_group(list(rs), backend=backend)
            if self._rank in rs:
                mine.append(self._groups[rs])
        return mine if axis == self.dp_axis else mine[0]

    def unit_dp_ranks(self, unit: int, tp_index: int) -> tuple[int, ...]:
        return tuple(sorted(set(int(r) for r in self._mesh[:, unit, tp_index])))

    def group_of(self, ranks: tuple[int, ...]):
        return self._groups[ranks]


class HeterogeneousPipelineStageManager:
    """Chain pipeline of the pipeline this rank belongs to."""

    def __init__(self, pg_mesh: HeterogeneousProcessGroupMesh, pipeline_axis: int = 1, num_layers_per_stage: list[int] | None = None):
        self.pg_mesh = pg_mesh
        self.pipeline_axis = pipeline_axis
        self.pipeline_index = pg_mesh.coords[0][pg_mesh.dp_axis]
        self.template = pg_mesh.pipelines[self.pipeline_index]
        self.my_modal = self.template
        self.is_interleave, self.num_model_chunks = False, 1
        tp_index = pg_mesh.coords[0][pg_mesh.tp_axis]
        # stage -> the rank at my tp index
        self.stage_ranks, unit = [], 0
        for modules in self.template.modules_per_stage:
            self.stage_ranks.append(int(pg_mesh.mesh[self.pipeline_index, unit, tp_index]))
            unit += len(modules)
        self._stage = self.stage_ranks.index(pg_mesh.rank)

    is_encoder = False

    @property
    def num_stages(self) -> int:
        return self.template.num_stages

    num_stages_in_modal = num_stages

    @property
    def stage(self) -> int:
        return self._stage

    stage_in_modal = stage

    def is_first_stage(self, ignore_chunk=False, check_only_in_modal=True) -> bool:
        return self._stage == 0

    def is_last_stage(self, ignore_chunk=False, check_only_in_modal=True) -> bool:
        return self._stage == self.num_stages - 1

    def get_prev_ranks(self) -> list[int]:
        return [self.stage_ranks[self._stage - 1]] if self._stage > 0 else [self.stage_ranks[-1]]

    def get_next_ranks(self) -> list[int]:
        return [self.stage_ranks[(self._stage + 1) % self.num_stages]]

    def get_prev_rank(self) -> int:
        return self.get_prev_ranks()[0]

    def get_next_rank(self) -> int:
        return self.get_next_ranks()[0]

    def held_module_names(self) -> list[str]:
        return list(self.template.modules_per_stage[self._stage])

    def distribute_layers(self, *a, **k) -> list[int]:
        return self.template.get_num_layers_per_stage()

    def get_stage_index(self, layers_per_stage: list[int], stage: int | None = None, **k) -> tuple[int, int]:
        stage = self._stage if stage is None else stage
        start = sum(layers_per_stage[:stage])
        return (start, start + layers_per_stage[stage])


class HeterogeneousBatchSampler(BatchSampler):
    """Pipeline ``i`` receives ``microbatch_size * num_microbatches[i]`` consecutive samples of every global batch."""

    def __init__(self, dataset: Dataset, pipeline_index: int, microbatch_size: int, num_microbatches: list[int],
                 shuffle: bool = True, seed: int = 0, drop_last: bool = False):
        if pipeline_index >= len(num_microbatches):
            raise IndexError(f"pipeline_index={pipeline_index} is out of range. Given number of microbatches={len(num_microbatches)}")
        self.dataset, self.microbatch_size = dataset, microbatch_size
        self.pipeline_index, self.num_microbatches = pipeline_index, num_microbatches
        self.epoch, self.drop_last = 0, True
        self.global_batch_size = microbatch_size * sum(num_microbatches)
        self.num_samples = math.floor(len(dataset) / self.global_batch_size)
        self.shuffle, self.seed = shuffle, seed

    def __iter__(self) -> Iterator[list[int]]:
        if self.shuffle:
            g = torch.Generator()
            g.manual_seed(self.seed + self.epoch)
            order = torch.randperm(self.num_samples, generator=g).tolist()
        else:
            order = list(range(self.num_samples))
        offset = sum(self.num_microbatches[: self.pipeline_index])
        count = self.num_microbatches[self.pipeline_index]
        for i in range(self.num_samples):
            start = order[i] * self.global_batch_size + self.microbatch_size * offset
            yield list(range(start, start + self.microbatch_size * count))

    def __len__(self) -> int:
        return self.num_samples

    def set_epoch(self, epoch: int):
        self.epoch = epoch


class HeterogeneousDataLoader(DataLoader):
    """A DataLoader that is created first and bound to a pipeline later (``configure``), once the plan is known."""

    def __init__(self, dataset: Dataset, global_batch_size: int = 1, microbatch_size: int = 1, shuffle: bool = False,
                 seed: int = 1024, **kwargs):
        assert global_batch_size % microbatch_size == 0, "global_batch_size must be divisible by microbatch_size."
        self.global_batch_size, self.microbatch_size = global_batch_size, microbatch_size
        self._shuffle, self._seed, self._kwargs, self._dataset = shuffle, seed, kwargs, dataset
        self.batch_sampler = None
        self._configured = False

    def configure(self, pipeline_index: int, num_microbatches: list[int]):
        assert self.global_batch_size == self.microbatch_size * sum(num_microbatches), (
            "inconsistent global batch size and numbers of micro-batches")
        sampler = HeterogeneousBatchSampler(self._dataset, pipeline_index, self.microbatch_size, num_microbatches,
                                            self._shuffle, self._seed)
        # (re-)binding after a re-plan: DataLoader refuses attribute changes once initialised
        object.__setattr__(self, "_DataLoader__initialized", False)
        super().__init__(self._dataset, batch_sampler=sampler, **self._kwargs)
        self._configured = True

    def __iter__(self):
        assert self._configured, "HeterogeneousDataLoader.configure() must be called before iterating"
        return super().__iter__()

    def __len__(self) -> int:
        assert self._configured, "HeterogeneousDataLoader.configure() must be called before len()"
        return len(self.batch_sampler)


class HeterogeneousParallelModule(nn.Module):
    def __init__(self, module: nn.Module, stage_manager: HeterogeneousPipelineStageManager, unit_dp_groups: dict,
                 tp_group, precision: str | None, device, loss_weight: float):
        super().__init__()
        self.module = module
        self.stage_manager = stage_manager
        self.unit_dp_groups = unit_dp_groups  # unit name -> process group (or None when held by one pipeline only)
        self.tp_group = tp_group
        self.loss_weight = loss_weight
        self.require_grad_sync = True
        self.optimizer = None
        dtype = PRECISION[precision]
        if dtype is not None:
            module.to(dtype)
        if device is not None:
            module.to(device)

    def unwrap(self):
        return self.module

    def forward(self, hidden_states=None, **kwargs):
        sm = self.stage_manager
        if not sm.is_first_stage():
            kwargs = {k: v for k, v in kwargs.items() if k not in ("input_ids", "inputs_embeds")}
            kwargs["hidden_states"] = hidden_states[0] if isinstance(hidden_states, (list, tuple)) else hidden_states
        if not sm.is_last_stage():
            kwargs.pop("labels", None)
        out = self.module(**kwargs)
        if not sm.is_last_stage():
            return {"hidden_states": out["hidden_states"]}
        return out

    def sync_shared_params(self):
        return None

    def sync_dp_grads(self):
        """Per pipeline unit, SUM the (already weighted) gradients over the pipelines that hold the unit."""
        for unit, group in self.unit_dp_groups.items():
            if group is None or dist.get_world_size(group) == 1:
                continue
            sub = self.module.get_submodule(unit) if unit else self.module
            for p in sub.parameters():
                g = getattr(p, "main_grad", None) if p.grad is None else p.grad
                if g is not None:
                    dist.all_reduce(g, group=group)

    def no_sync(self):
        from contextlib import nullcontext

        return nullcontext()


class HeterogeneousParallelPlugin:
    def __init__(self, tp_size: int = 1, microbatch_size: int = 1, precision: str | None = None, max_norm: float = 0.0,
                 enable_fused_normalization: bool = True, enable_flash_attention: bool = True, enable_jit_fused: bool = False,
                 parallel_output: bool = True, make_vocab_size_divisible_by: int = 64, device=None, **scaler_kwargs):
        self.tp_size, self.microbatch_size, self.precision, self.max_norm = tp_size, microbatch_size, precision, max_norm
        self.flags = dict(enable_fused_normalization=enable_fused_normalization, enable_flash_attention=enable_flash_attention,
                          enable_jit_fused=enable_jit_fused, parallel_output=parallel_output,
                          make_vocab_size_divisible_by=make_vocab_size_divisible_by)
        self.device = device
        self.scaler_kwargs = scaler_kwargs
        self.pipelines: list[PipelineTemplate] | None = None
        self.zero_stage = 0

    @property
    def train_batch_size(self) -> int:
        assert self.pipelines is not None, "call set_pipelines first"
        return self.global_batch_size

    def set_pipelines(self, pipelines: list[PipelineTemplate], num_microbatches: dict[PipelineTemplate, int] | list[int]):
        assert dist.is_initialized(), "torch.distributed is not initialized."
        assert pipelines and num_microbatches, "pipelines and num_microbatches must be specified together."
        counts = ([num_microbatches[p] for p in pipelines] if isinstance(num_microbatches, dict) else list(num_microbatches))
        n_ranks = sum(p.num_stages for p in pipelines) * self.tp_size
        assert dist.get_world_size() == n_ranks, (
            f"Number of ranks in pipeline templates ({n_ranks}) does not match world size ({dist.get_world_size()}).")
        self.pipelines, self.num_microbatches = pipelines, counts
        self.global_batch_size = self.microbatch_size * sum(counts)
        self.pg_mesh = HeterogeneousProcessGroupMesh(pipelines, self.tp_size)
        self._pipeline_index = self.pg_mesh.coords[0][0]
        self.stage_manager = HeterogeneousPipelineStageManager(self.pg_mesh)
        self.dp_groups = self.pg_mesh.get_group_along_axis(self.pg_mesh.dp_axis)
        self.tp_group = self.pg_mesh.get_group_along_axis(self.pg_mesh.tp_axis)
        self.pp_group = self.pg_mesh.get_group_along_axis(self.pg_mesh.pp_axis)
        self.dp_size = len(pipelines)
        if self.device is None:
            self.device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        self.schedule = MultimodalEncoderTrainingOneForwardOneBackwardSchedule(
            self.stage_manager, num_microbatches=counts[self._pipeline_index], microbatch_size=self.microbatch_size,
            device=self.device)

    def configure(self, model: nn.Module, optimizer=None, criterion: Callable | None = None, dataloader=None,
                  lr_scheduler=None, forced: bool = False):
        assert self.pipelines is not None, "call set_pipelines before boosting a model"
        if isinstance(model, HeterogeneousParallelModule):
            assert forced, "the model is already wrapped; pass forced=True to re-plan"
            model = model.module
        template = self.pipelines[self._pipeline_index]
        policy = policy_for_model(model)
        sc = ShardConfig(tensor_parallel_process_group=self.tp_group if self.tp_size > 1 else None,
                         pipeline_stage_manager=self.stage_manager, pipeline_template=template,
                         enable_tensor_parallelism=self.tp_size > 1,
                         extra_kwargs={"device": self.device, "dtype": PRECISION[self.precision]}, **self.flags)
        ShardFormer(sc).optimize(model, policy)
        names = type(policy).get_all_modules(model.config)
        tp_index = self.pg_mesh.coords[0][2]
        unit_groups = {}
        for unit_name in self.stage_manager.held_module_names():
            ranks = self.pg_mesh.unit_dp_ranks(names.index(unit_name), tp_index)
            unit_groups[unit_name] = self.pg_mesh.group_of(ranks) if len(ranks) > 1 else None
        weight = self.num_microbatches[self._pipeline_index] / sum(self.num_microbatches)
        wrapped = HeterogeneousParallelModule(model, self.stage_manager, unit_groups, self.tp_group if self.tp_size > 1 else None,
                                              self.precision, self.device, weight)
        if optimizer is not None:
            inner = optimizer.unwrap() if hasattr(optimizer, "unwrap") else optimizer
            params = [p for p in model.parameters() if p.requires_grad]
            cls = inner if isinstance(inner, type) else type(inner)
            defaults = {} if isinstance(inner, type) else dict(inner.defaults)
            if cls is FusedAdamW:
                kw = {k: defaults[k] for k in ("lr", "betas", "eps") if k in defaults}
                new = FusedAdamW(split_decay_groups(model, defaults.get("weight_decay", 0.01)), **kw)
            else:
                defaults.pop("differentiable", None)
                keep = {k: v for k, v in defaults.items() if k in cls.__init__.__code__.co_varnames}
                new = cls(params, **keep)
            optimizer = OptimizerWrapper(new, wrapped, self.max_norm, self.precision, self.tp_group if self.tp_size > 1 else None,
                                         self.pp_group, self.scaler_kwargs or None)
            wrapped.optimizer = optimizer
        if isinstance(dataloader, HeterogeneousDataLoader):
            dataloader.configure(self._pipeline_index, self.num_microbatches)
        return wrapped, optimizer, criterion, dataloader, lr_scheduler

    def execute_pipeline(self, data_iter: Iterator, model: HeterogeneousParallelModule, criterion: Callable, optimizer=None,
                         return_loss: bool = True, return_outputs: bool = False) -> dict:
        def weighted(out, batch):
            return criterion(out, batch) * (model.loss_weight)

        # loss per micro-batch / my micro-batches * (my micro-batches / all) = 1 / all micro-batches
        out = self.schedule.forward_backward_step(model, data_iter, weighted, optimizer, return_loss, return_outputs)
        if torch.is_grad_enabled() and optimizer is not None:
            model.sync_shared_params()
            model.sync_dp_grads()
        return out

    def prepare_dataloader(self, dataset, shuffle: bool = False, seed: int = 1024, **kwargs) -> HeterogeneousDataLoader:
        dl = HeterogeneousDataLoader(dataset, self.global_batch_size if self.pipelines else 1, self.microbatch_size, shuffle, seed, **kwargs)
        if self.pipelines is not None:
            dl.global_batch_size = self.global_batch_size
            dl.configure(self._pipeline_index, self.num_microbatches)
        return dl

    def get_checkpoint_io(self):
        return _HeteroCheckpointIO(self)

    def control_precision(self):
        return True

    def control_device(self):
        return True

    def support_no_sync(self):
        return True


class _HeteroCheckpointIO:
    """Pipeline 0 writes (its stages cover the whole model); every pipeline loads the units it holds."""

    def __init__(self, plugin: HeterogeneousParallelPlugin):
        self.plugin = plugin

    def _io(self, model):
        from .checkpoint_io import ModalParallelCheckpointIO

        pl = self.plugin
        io = ModalParallelCheckpointIO(None, model.tp_group, pl.pp_group, pl.stage_manager)
        io.dp_rank = pl._pipeline_index
        return io

    def save_model(self, model, checkpoint, shard=True, size_per_shard=1024, use_safetensors=True):
        self._io(model).save_sharded_model(model.module, checkpoint, size_per_shard, use_safetensors, merge_on_first=False)
        dist.barrier()
        from .checkpoint_io import MultimodalParallelCheckpointIO

        MultimodalParallelCheckpointIO._merge(model.module, checkpoint, self._io(model), use_safetensors)
        dist.barrier()

    def load_model(self, model, checkpoint, strict=False):
        self._io(model).load_sharded_model(model.module, checkpoint, strict)
        if model.optimizer is not None:
            model.optimizer.update_master_params()
        dist.barrier()
        return model

    def save_optimizer(self, optimizer, checkpoint, shard=True, size_per_shard=1024):
        # the replicas hold the same optimizer state after every step; pipeline 0 (all stages of it) writes, keyed by
        # parameter name, so a pipeline with another stage layout can read it back
        self._io(optimizer.model).save_sharded_optimizer(optimizer, optimizer.model.module, checkpoint, size_per_shard)
        dist.barrier()

    def load_optimizer(self, optimizer, checkpoint):
        self._io(optimizer.model).load_sharded_optimizer(optimizer, optimizer.model.module, checkpoint)
        dist.barrier()
