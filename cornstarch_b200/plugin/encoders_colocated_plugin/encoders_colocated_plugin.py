"""Encoders-colocated variant: every encoder lives on the SAME ranks and runs one after the other; the
pipeline is a plain chain ``[encoder stages..., LLM stages...]``.

Use it when encoders are small compared with the LLM, so that giving each its own ranks (modality
parallelism) would leave GPUs idle.  All encoders must share tensor-parallel size, sequence-parallel size
and number of stages.  An encoder rank at stage ``s`` holds stage ``s`` of every encoder and emits
``{"encoder_outputs_<key>": tensor}`` per encoder; the LLM's first stage merges them.  Mirrors the
reference plugin (cornstarch/plugin/encoders_colocated_plugin/: process_group_mesh.py:46-57,
encoders_colocated_stage_manager.py:16-305, one_f_one_b.py:20-126, encoders_colocated_plugin.py:50-411).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ...multimodal.modeling import ModalEncoderModule, MultimodalModel, _first_tensor
from ...parallel.mesh import MultiModalProcessGroupMesh
from ...parallel.schedule import MultimodalEncoderTrainingOneForwardOneBackwardSchedule
from ...parallel.stage_manager import MultiModalPipelineStageManager
from ...pipeline_template import PipelineTemplate
from ..modal_parallel_plugin import _FixedHeld
from ..multimodal_parallel_plugin import PRECISION, MultimodalParallelModule, MultimodalParallelPlugin, _Dropped, _DroppedLM


class EncodersColocatedProcessGroupMesh(MultiModalProcessGroupMesh):
    """Mesh of a chain: one pseudo-modality holding all encoders, then the LLM."""

    def __init__(self, encoder_templates: dict[PipelineTemplate, int | tuple[int, int]], llm_template, world_size=None, rank=None):
        sizes = [(v, 1) if isinstance(v, int) else tuple(v) for v in encoder_templates.values()]
        stages = [t.num_stages for t in encoder_templates]
        assert len(set(sizes)) == 1, "colocated encoders must share tp and sp sizes"
        assert len(set(stages)) == 1, "colocated encoders must have the same number of pipeline stages"
        merged = PipelineTemplate(
            "colocated_encoders",
            [[f"{i}:{m}" for i, t in enumerate(encoder_templates) for m in t.modules_per_stage[s]] for s in range(stages[0])])
        self.colocated_templates = list(encoder_templates.keys())
        self.merged_template = merged
        super().__init__({merged: sizes[0]}, llm_template, world_size, rank)


class EncodersColocatedPipelineStageManager(MultiModalPipelineStageManager):
    pass


class EncodersColocatedMultimodalParallelModule(MultimodalParallelModule):
    """Encoder ranks run every encoder (their stage of it); the LLM ranks behave as in the modality-parallel plugin."""

    def _forward_encoder(self, hidden_states=None, **kwargs):
        mm: MultimodalModel = self.module
        sm = self.stage_manager
        first = sm.is_first_stage(check_only_in_modal=True)
        last = sm.is_last_stage(check_only_in_modal=True)
        out = {}
        for key in mm.encoders_keys:
            enc: ModalEncoderModule = getattr(mm, f"{key}_encoder")
            name = f"encoder_outputs_{key}"
            if first:
                inputs = enc.preprocess_callback(inputs={k: v for k, v in kwargs.items()
                                                         if k in set(enc.forward_arg_names()) | set(enc.additional_args)})
                params = enc.forward_arg_names()
                if params[0] not in inputs:
                    continue
                res = enc.module(**{k: v for k, v in inputs.items() if k in params})
            else:
                inputs = kwargs
                if name not in kwargs:
                    continue
                params = enc.forward_arg_names()
                side = {k: v for k, v in kwargs.items() if k in params[1:] and k != "hidden_states" and v is not None}
                side.update({k[len(name) + 1 :]: v for k, v in kwargs.items() if k.startswith(name + ".")})
                res = enc.module(hidden_states=kwargs[name], **side)
            if not last:
                out[name] = res["hidden_states"]
                # what else the stage hands on (a relative-position bias, say) travels under "<name>.<key>"
                out.update({f"{name}.{k}": v for k, v in res.items() if k != "hidden_states" and isinstance(v, torch.Tensor)})
                continue
            res = enc.postprocess_module_callback(inputs=inputs, output=res)
            proj = enc.projector(_first_tensor(res), return_dict=True)
            proj = enc.postprocess_projector_callback(inputs=inputs, output=proj)
            out[name] = _first_tensor(proj)
        return out

    def forward(self, hidden_states=None, **kwargs):
        if self.my_modal_name != "language_model":
            return self._forward_encoder(hidden_states, **kwargs)
        sm = self.stage_manager
        if sm.is_first_stage(check_only_in_modal=True):
            mm = self.module
            hs = [kwargs.pop(f"encoder_outputs_{k}") for k in list(mm.encoders_keys) if f"encoder_outputs_{k}" in kwargs]
            return self._forward_llm(hs if hs else None, **kwargs)
        return self._forward_llm(hidden_states, **kwargs)


class EncodersColocatedMultimodalParallelPlugin(MultimodalParallelPlugin):
    def init_distributed(self):
        if self.distributed_initialized:
            return
        enc_templates = {pl.pipeline_template: (pl.tp_size, pl.sp_size) for pl in self.encoder_plugins.values()}
        llm = self.language_model_plugin
        self.pg_mesh = EncodersColocatedProcessGroupMesh(enc_templates, (llm.pipeline_template, llm.tp_size, llm.sp_size))
        M = self.pg_mesh
        self.stage_manager = EncodersColocatedPipelineStageManager(M, M.pp_axis)
        self.tp_group = M.get_group_along_axis(M.tp_axis)
        self.sp_group = M.get_group_along_axis(M.sp_axis)
        self.pp_groups = M.get_group_along_axis(M.pp_axis)
        M.get_group_along_axis([M.dp_axis, M.sp_axis])
        self.dp_group = M.get_group_along_axis(M.dp_axis)
        if isinstance(self.dp_group, list):
            self.dp_group = self.dp_group[0]
        self.dp_size = M.dp_size
        if self.device is None:
            self.device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        self.schedule = MultimodalEncoderTrainingOneForwardOneBackwardSchedule(
            self.stage_manager, self.num_microbatches, self.microbatch_size, device=self.device)
        self.distributed_initialized = True

    def my_modal_name(self) -> str:
        return "encoders" if self.stage_manager.is_encoder else "language_model"

    def configure(self, model: MultimodalModel, optimizer=None, criterion=None, dataloader=None, lr_scheduler=None):
        assert set(model.encoders_keys) == set(self.encoder_plugins), "every encoder of the model needs a plugin"
        self.init_distributed()
        sm = self.stage_manager
        dtype = PRECISION[self.precision]
        if sm.is_encoder:
            model.language_model = _DroppedLM(model.language_model.config)
            stage = sm.stage_in_modal
            params_holder = torch.nn.ModuleList()
            for key, plugin in self.encoder_plugins.items():
                enc = getattr(model, f"{key}_encoder")
                sc = plugin.make_shard_config(self.tp_group if plugin.tp_size > 1 else None,
                                              self.sp_group if plugin.sp_size > 1 else None,
                                              _FixedHeld(plugin.pipeline_template.modules_per_stage[stage]),
                                              device=self.device, dtype=dtype, **self.flags)
                plugin.configure(enc, sc, _FixedHeld(plugin.pipeline_template.modules_per_stage[stage]))
                if dtype is not None:
                    enc.to(dtype)
                enc.to(self.device)
                params_holder.append(enc)
            model.encoders_holder = params_holder  # all encoders = this rank's "modality"
            name, plugin = "encoders_holder", next(iter(self.encoder_plugins.values()))
        else:
            for key in model.encoders_keys:
                enc = getattr(model, f"{key}_encoder")
                enc.module = _Dropped(enc.module.config, enc.module)
                enc.projector = None
            plugin = self.language_model_plugin
            sc = plugin.make_shard_config(self.tp_group if plugin.tp_size > 1 else None,
                                          self.sp_group if plugin.sp_size > 1 else None, sm, device=self.device, dtype=dtype,
                                          **self.flags)
            plugin.configure(model.language_model, sc, sm)
            if getattr(plugin, "ep_size", 1) > 1:
                self._shard_experts(model.language_model, plugin)
            name = "language_model"
        wrapped = EncodersColocatedMultimodalParallelModule(model, name, sm, self.dp_group,
                                                            self.tp_group if plugin.tp_size > 1 else None,
                                                            self.sp_group if plugin.sp_size > 1 else None, self.precision,
                                                            self.device)
        if optimizer is not None:
            optimizer = self._wrap_optimizer(optimizer, wrapped, plugin)
            wrapped.optimizer = optimizer
        return wrapped, optimizer, criterion, dataloader, lr_scheduler


EncodersColocatedPlugin = EncodersColocatedMultimodalParallelPlugin
