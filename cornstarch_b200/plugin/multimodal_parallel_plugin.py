"""``MultimodalParallelPlugin``: modality-parallel pipeline + TP / CP / DP over a :class:`MultimodalModel`.

Every modality gets its own :class:`ModalParallelPlugin`; encoders run as separate pipeline branches on
disjoint ranks that feed the LLM's first stage (the signature feature of the reference,
cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:412-705).  The data-parallel
degree is inferred from the world size.  ``configure`` returns the wrapped model
(:class:`MultimodalParallelModule`), the wrapped optimizer, and passes criterion / dataloader /
scheduler through; ``execute_pipeline`` runs one global batch through the 1F1B schedule, then reduces
the gradients over the data-parallel group — on the flat gradient buffer of the fused optimizer, in a few
large buckets, instead of one blocking all-reduce per parameter (reference :362-384).
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Callable, Iterator

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader, DistributedSampler

from ..multimodal.modeling import ModalEncoderModule, MultimodalModel, _first_tensor
from ..ops import attention as A
from ..optim.fused_adamw import FusedAdamW, split_decay_groups
from ..optim.wrapper import OptimizerWrapper
from ..parallel.mesh import MultiModalProcessGroupMesh
from ..parallel.p2p import MultimodalPipelineP2PCommunication  # noqa: F401  (part of this module's public names)
from ..parallel.schedule import MultimodalEncoderTrainingOneForwardOneBackwardSchedule
from ..parallel.stage_manager import MultiModalPipelineStageManager
from .modal_parallel_plugin import ModalParallelPlugin

PRECISION = {None: None, "fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


class MultimodalParallelModule(nn.Module):
    """The model as seen by one rank: only its modality's held layers, with a pipeline-aware forward."""

    def __init__(self, module: MultimodalModel, my_modal_name: str, stage_manager, dp_group, tp_group, sp_group,
                 precision: str | None = None, device=None):
        super().__init__()
        self.module = module
        self.my_modal_name = my_modal_name
        self.stage_manager = stage_manager
        self.dp_group, self.tp_group, self.sp_group = dp_group, tp_group, sp_group
        self.require_grad_sync = True
        dtype = PRECISION[precision]
        mine = getattr(module, my_modal_name)
        if dtype is not None:
            mine.to(dtype)
        if device is not None:
            mine.to(device)
        self.optimizer: Any = None

    def unwrap(self) -> MultimodalModel:
        return self.module

    def set_modality_token_ids(self, token_ids: dict[str, int], new_num_tokens: int = 0):
        self.module.set_modality_token_ids(token_ids, new_num_tokens)

    def train(self, *a, **kw):
        self.module.train(*a, **kw)
        self.training = True
        return self

    # ------------------------------------------------------------------ forward per role
    def forward(self, hidden_states=None, **kwargs):
        if self.my_modal_name == "language_model":
            return self._forward_llm(hidden_states, **kwargs)
        return self._forward_encoder(hidden_states, **kwargs)

    def _forward_encoder(self, hidden_states=None, **kwargs):
        key = self.my_modal_name[: -len("_encoder")]
        enc: ModalEncoderModule = getattr(self.module, self.my_modal_name)
        sm = self.stage_manager
        first = sm is None or sm.is_first_stage(check_only_in_modal=True)
        last = sm is None or sm.is_last_stage(check_only_in_modal=True)
        if first:
            inputs = enc.preprocess_callback(inputs={k: v for k, v in kwargs.items()
                                                     if k in set(enc.forward_arg_names()) | set(enc.additional_args)})
            params = enc.forward_arg_names()
            out = enc.module(**{k: v for k, v in inputs.items() if k in params})
        else:
            inputs = kwargs
            if isinstance(hidden_states, (list, tuple)):
                hidden_states = hidden_states[0]
            # besides the hidden states a later stage gets what the stage before it handed on (a relative-position
            # bias, say) and the per-sample arguments of the micro-batch (an image grid), never the raw main input
            params = enc.forward_arg_names()
            side = {k: v for k, v in kwargs.items() if k in params[1:] and k != "hidden_states" and v is not None}
            out = enc.module(hidden_states=hidden_states, **side)
        if not last:
            return {k: v for k, v in out.items() if isinstance(v, torch.Tensor)}
        out = enc.postprocess_module_callback(inputs=inputs, output=out)
        proj = enc.projector(_first_tensor(out), return_dict=True)
        proj = enc.postprocess_projector_callback(inputs=inputs, output=proj)
        return {"hidden_states": _first_tensor(proj)}

    def _forward_llm(self, hidden_states=None, input_ids=None, attention_mask=None, labels=None, position_ids=None, **kwargs):
        mm = self.module
        lm = mm.language_model
        sm = self.stage_manager
        first = sm is None or sm.is_first_stage(check_only_in_modal=True)
        last = sm is None or sm.is_last_stage(check_only_in_modal=True)
        mask = mm.build_attn_mask(input_ids, attention_mask) if mm.token_ids else attention_mask
        llm_kwargs = dict(attention_mask=mask, position_ids=position_ids)
        if input_ids is not None:
            llm_kwargs["full_shape"] = tuple(input_ids.shape)  # later stages may hold token-sharded hidden states
        if first:
            enc_outs = {}
            if hidden_states is not None:
                hs = hidden_states if isinstance(hidden_states, (list, tuple)) else [hidden_states]
                # previous ranks are sorted by rank id == order of the encoders dict
                for k, t in zip(mm.encoders_keys, hs):
                    enc_outs[k] = (t,)
            if mm.token_ids:
                embeds, _bits = mm.merge_encoder_outputs(enc_outs, input_ids, None, attention_mask)
            else:
                embeds = lm.get_input_embeddings()(input_ids)
            llm_kwargs["inputs_embeds"] = embeds
        else:
            if isinstance(hidden_states, (list, tuple)):
                hidden_states = hidden_states[0]
            llm_kwargs["hidden_states"] = hidden_states
        if last and labels is not None and mm.token_ids:
            ignore = torch.zeros_like(labels, dtype=torch.bool)
            for tid in mm.token_ids.values():
                ignore |= input_ids == tid
            labels = torch.where(ignore, torch.full_like(labels, -100), labels)
        if last:
            llm_kwargs["labels"] = labels
        out = lm(**llm_kwargs)
        if not last:
            return {"hidden_states": out["hidden_states"]}
        return out

    # ------------------------------------------------------------------ gradient synchronisation
    @contextmanager
    def no_sync(self):
        old = self.require_grad_sync
        self.require_grad_sync = False
        try:
            yield
        finally:
            self.require_grad_sync = old

    def sync_shared_params(self):
        return None  # tied parameters across pipeline stages are not supported (as in the reference, :73-79)

    def sync_dp_grads(self, bucket_bytes: int = 256 << 20):
        """Average gradients over the data-parallel group (which includes the context-parallel ranks)."""
        g = self.dp_group
        if g is None or dist.get_world_size(g) == 1:
            return
        opt = self.optimizer.unwrap() if hasattr(self.optimizer, "unwrap") else self.optimizer
        if isinstance(opt, FusedAdamW) and opt.use_arena:
            if opt._sharded:
                return  # ZeRO-1: the reduce-scatter happens inside the optimizer step
            if opt.dp_group is None:
                opt.dp_group = g
            opt.reduce_dp_grads(bucket_bytes)  # peer-memory kernel when the buffers are peer-mapped, else NCCL buckets
            return
        ws = dist.get_world_size(g)
        for p in getattr(self.module, self.my_modal_name).parameters():
            if p.grad is None:
                continue
            if not getattr(p, "expert_parallel", False):
                dist.all_reduce(p.grad, group=g)
            # an expert's gradient already holds every rank's tokens, each from that rank's own mean loss: only the 1 / dp
            p.grad.div_(ws)

    def sync_sp_grads(self, grads=None):
        return None  # context-parallel ranks are part of the data-parallel reduction group


class MultimodalParallelPlugin:
    def __init__(self, encoder_plugins: dict[str, ModalParallelPlugin] | None = None,
                 language_model_plugin: ModalParallelPlugin | None = None, precision: str | None = None,
                 enable_fused_normalization: bool = True, enable_flash_attention: bool = True,
                 enable_jit_fused: bool = False, num_microbatches: int | None = None, microbatch_size: int | None = None,
                 initial_scale: float = 2**16, min_scale: float = 1, growth_factor: float = 2, backoff_factor: float = 0.5,
                 growth_interval: int = 1000, hysteresis: int = 2, max_scale: float = 2**32, max_norm: float = 0,
                 parallel_output: bool = True, make_vocab_size_divisible_by: int = 64, zero_stage: int = 0,
                 grad_dtype: torch.dtype = torch.bfloat16, device=None, overlap_p2p: bool | None = None):
        assert language_model_plugin is not None, "a language model plugin is required"
        # Pipeline messages posted asynchronously (sends not waited for, receives posted ahead of the compute they
        # overlap with).  None = on for NCCL (every pipeline edge gets one two-rank process group per message
        # direction), off for gloo; CORNSTARCH_B200_OVERLAP_P2P=0/1 overrides.
        self.overlap_p2p = overlap_p2p
        for name, pl in {**(encoder_plugins or {}), "language_model": language_model_plugin}.items():
            assert pl.pipeline_template is not None, f"A pipeline template must be specified for {name} (the plugin always pipelines)."
        self.encoder_plugins = dict(encoder_plugins or {})
        self.language_model_plugin = language_model_plugin
        self.precision = precision
        self.flags = dict(enable_fused_normalization=enable_fused_normalization, enable_flash_attention=enable_flash_attention,
                          enable_jit_fused=enable_jit_fused, parallel_output=parallel_output,
                          make_vocab_size_divisible_by=make_vocab_size_divisible_by)
        self.num_microbatches, self.microbatch_size = num_microbatches, microbatch_size
        self.scaler_kwargs = dict(initial_scale=initial_scale, min_scale=min_scale, growth_factor=growth_factor,
                                  backoff_factor=backoff_factor, growth_interval=growth_interval, hysteresis=hysteresis,
                                  max_scale=max_scale)
        self.max_norm = max_norm
        self.zero_stage = zero_stage
        self.grad_dtype = grad_dtype
        self.device = device
        self.distributed_initialized = False

    # ------------------------------------------------------------------ groups
    def init_distributed(self):
        if self.distributed_initialized:
            return
        enc_templates = {pl.pipeline_template: (pl.tp_size, pl.sp_size) for pl in self.encoder_plugins.values()}
        llm = self.language_model_plugin
        self.pg_mesh = MultiModalProcessGroupMesh(enc_templates, (llm.pipeline_template, llm.tp_size, llm.sp_size))
        M = self.pg_mesh
        self.stage_manager = MultiModalPipelineStageManager(M, M.pp_axis)
        self.tp_group = M.get_group_along_axis(M.tp_axis)
        self.sp_group = M.get_group_along_axis(M.sp_axis)
        self.pp_groups = M.get_group_along_axis(M.pp_axis)
        my_sp = self._my_plugin().sp_size
        if my_sp > 1:
            # context-parallel ranks hold different tokens of the same samples: they average gradients with dp
            self.dp_group = M.get_group_along_axis([M.dp_axis, M.sp_axis])
        else:
            M.get_group_along_axis([M.dp_axis, M.sp_axis])  # created collectively on every rank
            self.dp_group = M.get_group_along_axis(M.dp_axis)
        if isinstance(self.dp_group, list):
            self.dp_group = self.dp_group[0]
        self.dp_size = M.dp_size
        if self.device is None:
            self.device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        import os

        overlap = self.overlap_p2p
        env = os.environ.get("CORNSTARCH_B200_OVERLAP_P2P")
        if env is not None:
            overlap = env == "1"
        if overlap is None:
            # A receive that was posted ahead is an NCCL kernel that stays on the GPU until its sender has sent.  The fused
            # tensor- / context- / expert-parallel kernels are persistent (one thread block per SM) and wait for their peers
            # inside the kernel: they need every thread block resident at once.  With a pending receive holding SMs on
            # both ranks of a pair, each rank's late blocks wait for an SM that the other rank's waiting blocks hold, and
            # every such launch runs into its bounded wait (measured: 2 s per fused GEMM on 4 GPUs).  So the overlap is on
            # by default only where no such kernel runs: every modality without tensor, context or expert parallelism.
            plugins = list(self.encoder_plugins.values()) + [self.language_model_plugin]
            peer_kernels = any(getattr(pl, "tp_size", 1) > 1 or getattr(pl, "sp_size", 1) > 1 or getattr(pl, "ep_size", 1) > 1
                               for pl in plugins if pl is not None)
            overlap = dist.get_backend() == "nccl" and not peer_kernels
        edge_groups = None
        if overlap:
            from ..parallel.p2p import make_edge_groups

            sm = self.stage_manager
            nxt = [] if sm.is_last_stage(check_only_in_modal=False) else sm.get_next_ranks()
            edge_groups = make_edge_groups(nxt)  # collective over all ranks: two groups per pipeline edge
        self.schedule = MultimodalEncoderTrainingOneForwardOneBackwardSchedule(
            self.stage_manager, self.num_microbatches, self.microbatch_size, device=self.device, overlap_p2p=bool(overlap),
            p2p_edge_groups=edge_groups)
        self.distributed_initialized = True

    def my_modal_name(self) -> str:
        modal = self.stage_manager.my_modal
        for name, pl in self.encoder_plugins.items():
            if pl.pipeline_template == modal:
                return f"{name}_encoder"
        return "language_model"

    def _my_plugin(self) -> ModalParallelPlugin:
        name = self.my_modal_name()
        return self.language_model_plugin if name == "language_model" else self.encoder_plugins[name[: -len("_encoder")]]

    # ------------------------------------------------------------------ configure
    def configure(self, model: MultimodalModel, optimizer=None, criterion: Callable | None = None,
                  dataloader: DataLoader | None = None, lr_scheduler=None):
        assert isinstance(model, MultimodalModel), "MultimodalParallelPlugin works on a MultimodalModel"
        assert set(model.encoders_keys) == set(self.encoder_plugins), "every encoder of the model needs a plugin"
        self.init_distributed()
        name = self.my_modal_name()
        dtype = PRECISION[self.precision]
        # drop the modalities this rank does not run
        for key in model.encoders_keys:
            if f"{key}_encoder" != name:
                enc = getattr(model, f"{key}_encoder")
                enc.module = _Dropped(enc.module.config, enc.module)
                enc.projector = None
        if name != "language_model":
            model.language_model = _DroppedLM(model.language_model.config)
        plugin = self._my_plugin()
        sc = plugin.make_shard_config(self.tp_group if plugin.tp_size > 1 else None,
                                      self.sp_group if plugin.sp_size > 1 else None,
                                      self.stage_manager, device=self.device, dtype=dtype, **self.flags)
        plugin.configure(getattr(model, name), sc, self.stage_manager)
        if getattr(plugin, "ep_size", 1) > 1:
            self._shard_experts(getattr(model, name), plugin)
        wrapped = MultimodalParallelModule(model, name, self.stage_manager, self.dp_group,
                                           self.tp_group if plugin.tp_size > 1 else None,
                                           self.sp_group if plugin.sp_size > 1 else None, self.precision, self.device)
        if optimizer is not None:
            optimizer = self._wrap_optimizer(optimizer, wrapped, plugin)
            wrapped.optimizer = optimizer
        return wrapped, optimizer, criterion, dataloader, lr_scheduler

    def _shard_experts(self, module, plugin: ModalParallelPlugin) -> None:
        """Expert parallelism of a MoE modality: every sparse block this rank holds keeps ``experts / ep`` experts, tokens
        travel between the data-parallel ranks of this stage (``parallel/ep.py``).  The expert parameters are then not
        replicated over that group: the gradient reduction skips them and the optimizer only rescales them."""
        from ..parallel.ep import shard_experts

        dp = dist.get_world_size(self.dp_group) if self.dp_group is not None else 1
        assert plugin.ep_size == dp, (
            f"ep_size {plugin.ep_size} must equal the data-parallel degree {dp}: experts are sharded over the data-parallel ranks")
        assert plugin.sp_size == 1, "expert parallelism over ranks that also split the sequence is not supported"
        params = shard_experts(module, self.dp_group, capacity_factor=plugin.ep_capacity_factor,
                               capacity_tokens=getattr(plugin, "ep_capacity_tokens", None))
        assert params or not any(hasattr(m, "experts") for m in module.modules()), "no sparse MoE block found to shard"

    def _wrap_optimizer(self, optimizer, wrapped: MultimodalParallelModule, plugin: ModalParallelPlugin):
        """Rebuild the optimizer over the parameters that survived sharding (same class and hyper-parameters)."""
        mine = getattr(wrapped.module, wrapped.my_modal_name)
        params = [p for p in mine.parameters() if p.requires_grad]
        if isinstance(optimizer, type):
            cls, defaults = optimizer, {}
        else:
            cls, defaults = type(optimizer), dict(optimizer.defaults)
        if cls is FusedAdamW or (cls in (torch.optim.AdamW, torch.optim.Adam) and params and params[0].is_cuda
                                 and params[0].dtype == torch.bfloat16):
            kw = {k: defaults[k] for k in ("lr", "betas", "eps", "weight_decay") if k in defaults}
            wd = kw.pop("weight_decay", 0.01 if cls is not torch.optim.Adam else 0.0)
            inner = FusedAdamW(split_decay_groups(mine, wd), grad_dtype=self.grad_dtype, zero_stage=self.zero_stage,
                               dp_group=self.dp_group, expert_group=self.dp_group if plugin.ep_size > 1 else None, **kw)
        else:
            defaults.pop("differentiable", None)
            keep = {k: v for k, v in defaults.items() if k in cls.__init__.__code__.co_varnames}
            inner = cls(params, **keep) if params else cls([torch.nn.Parameter(torch.zeros(1, device=self.device))], **keep)
        pp_group = self.pp_groups[0] if self.pp_groups else None
        opt = OptimizerWrapper(inner, wrapped, self.max_norm, self.precision, self.tp_group if plugin.tp_size > 1 else None,
                               pp_group, self.scaler_kwargs)
        opt.expert_group = self.dp_group if plugin.ep_size > 1 else None
        return opt

    # ------------------------------------------------------------------ data
    def prepare_dataloader(self, dataset, batch_size, shuffle=False, seed=1024, drop_last=False, pin_memory=False,
                           num_workers=0, distributed_sampler_cls=None, **kwargs) -> DataLoader:
        """Every rank of a data-parallel replica reads the same samples; replicas read disjoint shards."""
        self.init_distributed()
        M = self.pg_mesh
        dp_rank = M.coords[0][M.dp_axis]
        cls = distributed_sampler_cls or DistributedSampler
        sampler = cls(dataset, num_replicas=self.dp_size, rank=dp_rank, shuffle=shuffle, seed=seed, drop_last=drop_last)
        return DataLoader(dataset, batch_size=batch_size, sampler=sampler, drop_last=drop_last, pin_memory=pin_memory,
                          num_workers=num_workers, **kwargs)

    # ------------------------------------------------------------------ one step
    def execute_pipeline(self, data_iter: Iterator, model: MultimodalParallelModule, criterion: Callable,
                         optimizer=None, return_loss: bool = True, return_outputs: bool = False) -> dict:
        with model.no_sync():
            out = self.schedule.forward_backward_step(model, data_iter, criterion, optimizer, return_loss, return_outputs)
        if torch.is_grad_enabled() and optimizer is not None:
            model.sync_shared_params()
            model.sync_dp_grads()
        return out

    def get_checkpoint_io(self):
        from .checkpoint_io import MultimodalParallelCheckpointIO

        return MultimodalParallelCheckpointIO(self)

    def control_precision(self) -> bool:
        return True

    def control_device(self) -> bool:
        return True

    def support_no_sync(self) -> bool:
        return True


class _Dropped(nn.Module):
    """Stands where a modality's module was on ranks that do not run it (keeps the config for bookkeeping)."""

    def __init__(self, config, original=None):
        super().__init__()
        self.config = config
        self._forward_args = None
        if original is not None:
            import inspect

            self._forward_args = [k for k in inspect.signature(original.forward).parameters if k not in ("self", "kw", "kwargs")]

    def forward(self, *a, **k):
        raise RuntimeError("this modality is not executed on this rank")


class _DroppedLM(_Dropped):
    def get_input_embeddings(self):
        raise RuntimeError("the language model is not executed on this rank")
