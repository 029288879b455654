"""Multi-GPU trainer for ``bench.py``: the modality-parallel pipeline through ``Booster`` / ``MultimodalParallelPlugin``.

Plans per GPU count (``--parallelism auto``): the headline configuration is 8 GPUs = one encoder stage plus
three LLM stages with tensor parallelism 2 in every stage:

    8 GPUs: encoder stage + 3 LLM stages, tp 2 (the named configuration)
    2 / 4 GPUs: data parallel (every GPU holds the whole model; gradients reduced by the peer-memory kernel), which is
    faster there than a pipeline whose encoder stage would leave a GPU almost idle; the pipeline shapes remain
    available as explicit plans (``enc1+llm1xtp1``, ``enc1+llm3xtp1``).

An explicit plan is written ``enc<E>+llm<L>xtp<T>`` (e.g. ``enc1+llm3xtp2``); remaining ranks become data parallel.
"""

from __future__ import annotations

import re

import torch
import torch.distributed as dist

from .booster import Booster
from .optim.fused_adamw import FusedAdamW
from .pipeline_template import PipelineTemplate
from .plugin.modal_parallel_plugin import ModalParallelPlugin
from .plugin.multimodal_parallel_plugin import MultimodalParallelPlugin
from .zoo import SHAPES, build_model, synthetic_batch

AUTO = {2: (1, 1, 1), 4: (1, 3, 1), 8: (1, 3, 2)}


def parse_plan(plan: str, world: int) -> tuple[int, int, int]:
    if plan == "auto":
        assert world in AUTO, f"no automatic plan for {world} GPUs"
        return AUTO[world]
    m = re.fullmatch(r"enc(\d+)\+llm(\d+)xtp(\d+)", plan)
    assert m, f"cannot parse parallelism '{plan}'"
    return int(m.group(1)), int(m.group(2)), int(m.group(3))


class PipelineTrainer:
    def __init__(self, args, rank: int, world: int, device):
        from .bench_support import _model_name

        self.shape = SHAPES[args.shape]
        self.model_name = _model_name(args.shape)
        self.seq_len = self.shape.seq_len
        enc_stages, llm_stages, tp = parse_plan(args.parallelism, world)
        ranks_per_replica = (enc_stages * len([1 for _ in (self.shape.vision, self.shape.audio) if _]) + llm_stages) * tp
        assert world % ranks_per_replica == 0
        dp = world // ranks_per_replica
        self.parallelism = f"enc{enc_stages}+llm{llm_stages} x tp{tp} x dp{dp} (modality-parallel 1F1B)"
        self.global_batch = args.samples_per_gpu * world
        per_replica = self.global_batch // dp
        self.microbatch = args.microbatch
        self.device = device
        torch.manual_seed(1234)
        model = build_model(args.shape, device="meta", dtype=torch.bfloat16)
        model.gradient_checkpointing_enable()
        enc_plugins = {}
        for key in model.encoders_keys:
            enc = getattr(model, f"{key}_encoder")
            enc_plugins[key] = ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(enc, enc_stages))
        llm_plugin = ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(model.language_model, llm_stages))
        self.plugin = MultimodalParallelPlugin(encoder_plugins=enc_plugins, language_model_plugin=llm_plugin,
                                               precision="bf16", microbatch_size=args.microbatch, max_norm=1.0, device=device)
        self.booster = Booster(plugin=self.plugin)
        opt = FusedAdamW  # rebuilt over the held parameters by the plugin
        self.model, self.opt, self.criterion, *_ = self.booster.boost(model, opt, criterion=lambda out, batch: out.loss)
        self.model.train()
        self.opt.unwrap().param_groups[0]["lr"] = 1e-4
        M = self.plugin.pg_mesh
        dp_rank = M.coords[0][M.dp_axis]
        self.host = synthetic_batch(args.shape, per_replica, seed=77 + dp_rank, dtype=torch.bfloat16, pin=True)
        self.dev = {k: v.to(device) for k, v in self.host.items()}
        self.tokens_per_step = self.global_batch * self.seq_len
        self.h2d_bytes_per_step = sum(v.numel() * v.element_size() for v in self.host.values())
        self.d2h_bytes_per_step = 4
        self.is_last = self.plugin.stage_manager.is_last_stage(check_only_in_modal=False)
        sm = self.plugin.stage_manager
        self.role = f"{self.model.my_modal_name} stage {sm.stage_in_modal + 1}/{sm.num_stages_in_modal}, tp rank {M.coords[0][M.tp_axis]}"

    def _step(self, batch):
        out = self.booster.execute_pipeline(iter([batch]), self.model, self.criterion, self.opt, return_loss=True)
        self.opt.step()
        self.opt.zero_grad()
        return out["loss"]

    recompute = "every layer"

    def checks(self) -> dict:
        """Agreement of replicated parameters inside this rank's data-parallel and tensor-parallel groups after the timed
        steps; every rank reports, the values are combined over all ranks by the caller."""
        from .bench_support import replica_checks
        from .plugin.checkpoint_io import _tp_info

        inner = getattr(self.model.module, self.model.my_modal_name)
        tp = self.plugin.tp_group[0] if isinstance(self.plugin.tp_group, list) else self.plugin.tp_group
        tp = tp if (tp is not None and dist.get_world_size(tp) > 1) else None
        return replica_checks(list(inner.named_parameters()), dp_group=self.model.dp_group, tp_group=tp,
                              tp_sharded=set(_tp_info(inner)))

    def tune_recompute(self):
        """Call after each of the first two steps: decoder layers that fit in the memory left over stop being recomputed (per stage; the
        tensor-parallel peers agree on the number)."""
        from .utils.recompute import RecomputeTuner

        sm = self.plugin.stage_manager
        is_llm = self.model.my_modal_name == "language_model"
        llm_stages = self.plugin.language_model_plugin.pipeline_template.num_stages
        in_flight = llm_stages - sm.stage_in_modal if is_llm else 1
        tp = self.plugin.language_model_plugin.tp_size
        if getattr(self, "_tuner", None) is None:
            self._tuner = RecomputeTuner(self.model.module, self.microbatch * self.seq_len, tp, in_flight,
                                         self.plugin.tp_group if tp > 1 else None)
        keep = self._tuner.after_step() if is_llm else 0
        counts = [None] * dist.get_world_size()
        dist.all_gather_object(counts, (is_llm, keep))
        kept = [k for llm, k in counts if llm]
        self.recompute = f"decoder layers kept without recomputation per LLM rank: {kept}; encoder layers recomputed"
        return keep

    def step_device(self):
        return self._step(self.dev)

    def step_e2e(self) -> float:
        batch = {k: v.to(self.device, non_blocking=True) for k, v in self.host.items()}
        loss = self._step(batch)
        return float(loss.item()) if loss is not None else float("nan")
