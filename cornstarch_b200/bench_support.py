"""Trainer objects used by ``bench.py``: the same public calls a user script makes, packaged per parallel plan.

* 1 GPU: ``MultimodalModel`` + ``FusedAdamW`` in a plain loop with gradient accumulation.
* N GPUs: ``Booster(plugin=MultimodalParallelPlugin(...))`` and ``booster.execute_pipeline`` (modality-parallel
  pipeline with tensor parallelism), or plain data parallelism when asked for.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .optim.fused_adamw import FusedAdamW, split_decay_groups
from .utils.recompute import RecomputeTuner, activation_bytes_per_layer, tune_recompute  # noqa: F401  (also imported from here)
from .zoo import SHAPES, build_model, synthetic_batch


def replica_checks(named_params, dp_group=None, tp_group=None, tp_sharded: set | None = None) -> dict:
    """Bit-level agreement of parameters that must be identical on several ranks, after the timed steps.

    Every parameter is reduced to a 64-bit checksum of its bit pattern (sum of its 16-bit words as integers) on the
    device; the checksum vectors are gathered and compared.  ``dp``: all parameters over the data-parallel group;
    ``tp_replicated``: the parameters that tensor parallelism does not shard (norm weights, biases of row-parallel
    layers) over the tensor-parallel group.  Values: number of parameters compared and how many of them differ."""
    named = [(n, p) for n, p in named_params if p is not None and p.numel() > 0]
    out = {}

    def sums(items):
        if not items:
            return torch.zeros(0, dtype=torch.int64, device="cuda" if torch.cuda.is_available() else "cpu")
        return torch.stack([p.detach().contiguous().view(torch.int16 if p.element_size() == 2 else torch.int32)
                            .to(torch.int64).sum() for _, p in items])

    for key, group, items in (("dp", dp_group, named),
                              ("tp_replicated", tp_group, [(n, p) for n, p in named if n not in (tp_sharded or set())])):
        if group is None or dist.get_world_size(group) < 2:
            continue
        mine = sums(items)
        everyone = [torch.empty_like(mine) for _ in range(dist.get_world_size(group))]
        dist.all_gather(everyone, mine, group=group)
        bad = int(sum((e != everyone[0]).sum() for e in everyone[1:]))
        out[key] = {"ranks": dist.get_world_size(group), "params": len(items), "mismatched": bad}
    return out


class SingleDeviceTrainer:
    parallelism = "single"

    def checks(self) -> dict:
        """Replica agreement after the timed steps (see :func:`replica_checks`); expert-parallel parameters differ by design."""
        if self.world < 2:
            return {}
        named = [(n, p) for n, p in self.model.named_parameters() if not getattr(p, "expert_parallel", False)]
        return replica_checks(named, dp_group=self.dp_group)

    def __init__(self, shape: str, samples_per_step: int, microbatch: int, device, lr: float = 1e-4, seed: int = 0,
                 dp_group=None, mask_mode: str = "modality", dtype=torch.bfloat16):
        self.shape = SHAPES[shape]
        self.model_name = _model_name(shape)
        self.seq_len = self.shape.seq_len
        self.samples = samples_per_step
        self.microbatch = microbatch
        self.device = device
        self.dp_group = dp_group
        self.world = dist.get_world_size(dp_group) if dp_group is not None else 1
        torch.manual_seed(seed)
        self.model = build_model(shape, device=device, dtype=dtype, mask_mode=mask_mode)
        self.model.gradient_checkpointing_enable()
        self.model.train()
        self.opt = self.make_optimizer(lr)
        self.n_micro = samples_per_step // microbatch
        rank = self.data_rank()
        self.host = [synthetic_batch(shape, microbatch, seed=1000 * rank + i, dtype=dtype, pin=True)
                     for i in range(self.n_micro)]
        self.dev = [{k: v.to(device) for k, v in b.items()} for b in self.host]
        self.global_batch = samples_per_step * self.world
        self.tokens_per_step = self.global_batch * self.seq_len
        self.h2d_bytes_per_step = sum(v.numel() * v.element_size() for b in self.host for v in b.values())
        self.d2h_bytes_per_step = 4
        if self.world > 1:
            self.parallelism = f"dp{self.world}"

    def make_optimizer(self, lr):
        from .ops import _native as nat

        if nat.LIBRARY_MODE:
            return _TorchAdamW(self.model, lr)
        return FusedAdamW(split_decay_groups(self.model, 0.01), lr=lr, max_norm=1.0, dp_group=self.dp_group)

    def data_rank(self) -> int:
        return dist.get_rank(self.dp_group) if self.dp_group is not None else 0

    def reduce_grads(self):
        if self.world > 1 and self.opt.use_arena and self.opt.reduce_dp_grads():
            return
        if self.world > 1:
            for g in self.opt.flat_grads() if self.opt.use_arena else [p.grad for p in self.model.parameters() if p.grad is not None]:
                dist.all_reduce(g, op=dist.ReduceOp.SUM if dist.get_backend(self.dp_group) == "gloo" else dist.ReduceOp.AVG,
                                group=self.dp_group)
                if dist.get_backend(self.dp_group) == "gloo":
                    g.div_(self.world)

    def _run(self, batches):
        import contextlib

        total = None
        for i, b in enumerate(batches):
            # the last micro-batch's backward pass overlaps the gradient reduction of the layers it has finished
            last = i == len(batches) - 1 and self.world > 1 and self.overlap_reduce and hasattr(self.opt, "overlapped_reduce")
            with (self.opt.overlapped_reduce() if last else contextlib.nullcontext()):
                out = self.model(**b)
                loss = out.loss / self.n_micro
                loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        self.reduce_grads()
        self.opt.step()
        self.opt.zero_grad()
        return total

    recompute = "every layer"
    overlap_reduce = True

    def tune_recompute(self):
        """Call after each of the first two steps: layers that fit in the memory left over stop being recomputed."""
        from .ops import _native as nat

        if getattr(self, "_tuner", None) is None:
            self._tuner = RecomputeTuner(self.model, self.microbatch * self.seq_len, 1, 1, self.dp_group)
        keep = self._tuner.after_step()
        n = len(self.model.language_model.model.layers)
        self.recompute = f"{n - keep} of {n} decoder layers (the other {keep} fit in free memory), encoder layers"
        return keep

    def recompute_everything(self):
        """Back to recomputing every layer (after an out-of-memory error): drops half-accumulated gradients too."""
        self.model.gradient_checkpointing_enable({"keep_last_layers": 0})
        self.recompute = "every layer (a step with kept layers ran out of memory)"
        self.opt.zero_grad()
        if getattr(self.opt, "use_arena", False):
            self.opt.clear_main_grads()
        torch.cuda.empty_cache()

    def step_device(self):
        return self._run(self.dev)

    def step_e2e(self) -> float:
        batches = [{k: v.to(self.device, non_blocking=True) for k, v in b.items()} for b in self.host]
        return float(self._run(batches).item())


class _TorchAdamW(torch.optim.AdamW):
    """Library baseline optimizer: ``torch.optim.AdamW(fused=True)`` with global-norm clipping, no flat arena."""

    use_arena = False

    def __init__(self, model, lr):
        self._params = [p for p in model.parameters() if p.requires_grad]
        super().__init__(split_decay_groups(model, 0.01), lr=lr, fused=True)

    def step(self, closure=None):
        torch.nn.utils.clip_grad_norm_(self._params, 1.0)
        return super().step(closure)

    def reduce_dp_grads(self):
        return False

    def flat_grads(self):
        return [p.grad for p in self._params if p.grad is not None]


class ExpertParallelTrainer(SingleDeviceTrainer):
    """Data parallel over all ranks; the experts of every MoE layer are sharded over the same ranks (expert parallel,
    dispatch / combine all-to-all); replicated parameters use ZeRO-1 (optimizer state sharded, gradients reduce-scattered)."""

    def __init__(self, shape, samples_per_step, microbatch, device, group, **kw):
        self.group = group
        super().__init__(shape, samples_per_step, microbatch, device, dp_group=group, **kw)
        self.parallelism = f"dp{self.world} + ep{self.world} (expert all-to-all) + ZeRO-1"
        if self.ep_capacity:
            self.parallelism += f", capacity factor {self.ep_capacity} (static shapes, no host synchronisation)"

    def make_optimizer(self, lr):
        from .parallel.ep import shard_experts

        import os

        cap = os.environ.get("CORNSTARCH_B200_EP_CAPACITY")  # e.g. 1.25: static-shape dispatch without host reads
        self.ep_capacity = float(cap) if cap else None
        shard_experts(self.model.language_model, self.group, capacity_factor=self.ep_capacity)
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
        return FusedAdamW(split_decay_groups(self.model, 0.01), lr=lr, max_norm=1.0, zero_stage=1, dp_group=self.group,
                          expert_group=self.group)

    def reduce_grads(self):
        if self.opt.use_arena:
            return  # ZeRO-1 reduce-scatters inside the step; expert gradients are not replicated
        ws = self.world
        for p in self.model.parameters():
            if p.grad is None:
                continue
            if getattr(p, "expert_parallel", False):
                p.grad.div_(ws)
            else:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(ws)


class ContextParallelTrainer(SingleDeviceTrainer):
    """One replica over all ranks: every rank holds the whole model and 1/cp of every sequence (gathered-KV context
    parallelism with makespan-balanced token assignment); gradients are averaged over the context-parallel ranks, which
    is also where ZeRO-1 shards the optimizer state."""

    def __init__(self, shape, samples_per_step, microbatch, device, group, **kw):
        self.group = group
        super().__init__(shape, samples_per_step, microbatch, device, dp_group=group, mask_mode="instance", **kw)
        self.global_batch = samples_per_step  # all ranks work on the same samples
        self.tokens_per_step = self.global_batch * self.seq_len
        self.parallelism = f"cp{self.world} (gathered-KV ring attention, makespan_min) + ZeRO-1"

    def data_rank(self) -> int:
        return 0  # same data on every rank

    def make_optimizer(self, lr):
        from .models.llama import ParallelContext
        from .parallel.cp import install_context_parallel_attention

        install_context_parallel_attention(self.model.language_model, self.group)
        self.model.language_model.set_parallel_context(
            ParallelContext(sp_group=self.group, sp_mode="ring_attn", cp_dist_mode="makespan_min"))
        return FusedAdamW(split_decay_groups(self.model, 0.01), lr=lr, max_norm=1.0, zero_stage=1, dp_group=self.group)

    def reduce_grads(self):
        if self.opt.use_arena:
            return
        super().reduce_grads()


class TensorParallelTrainer(SingleDeviceTrainer):
    """One replica over all ranks: the language model is tensor parallel over the group (replicated activations, or
    token-sharded ones with ``CORNSTARCH_B200_TP_SEQ_SHARD=1``) and so are the encoder and its projector; every rank
    sees the same data.  Used to measure the two tensor-parallel layouts inside a whole training step
    (``bench.py --parallelism tp``)."""

    def __init__(self, shape, samples_per_step, microbatch, device, group, **kw):
        self.group = group
        super().__init__(shape, samples_per_step, microbatch, device, dp_group=None, **kw)
        self.world = dist.get_world_size(group)
        self.global_batch = samples_per_step  # all ranks work on the same samples
        self.tokens_per_step = self.global_batch * self.seq_len
        import os

        sharded = os.environ.get("CORNSTARCH_B200_TP_SEQ_SHARD", "0") == "1"
        self.parallelism = f"tp{self.world} ({'token-sharded' if sharded else 'replicated'} activations)"

    def data_rank(self) -> int:
        return 0  # same data on every rank

    def make_optimizer(self, lr):
        from .ops import _native as nat
        from .shardformer.shard.shard_config import ShardConfig
        from .shardformer.shard.shardformer import ShardFormer

        sc = ShardConfig(tensor_parallel_process_group=self.group, enable_tensor_parallelism=True, extra_kwargs={"device": self.device})
        ShardFormer(sc).optimize(self.model.language_model)
        # the encoders (with their projectors) are tensor parallel as well: replicas that compute the same gradients
        # independently would drift apart in the last bit (dQ of the attention backward is summed in no fixed order)
        for key in self.model.encoders_keys:
            ShardFormer(sc).optimize(getattr(self.model, f"{key}_encoder"))
        if nat.LIBRARY_MODE:
            return _TorchAdamW(self.model, lr)
        return FusedAdamW(split_decay_groups(self.model, 0.01), lr=lr, max_norm=1.0, norm_groups=[self.group])

    def reduce_grads(self):
        return  # no data parallelism: replicated parts see identical data, sharded parts are reduced inside the layers

    def checks(self) -> dict:
        from .plugin.checkpoint_io import _tp_info

        return replica_checks(list(self.model.named_parameters()), tp_group=self.group, tp_sharded=set(_tp_info(self.model)))


def _model_name(shape: str) -> str:
    return {
        "vlm": "SigLIP-so400m-shape (27L,h1152) + MLP projector + Llama-3.1-8B-shape (32L,h4096,vocab 128256)",
        "valm": "SigLIP-so400m-shape + Whisper-large-v3-shape + Llama-3.1-8B-shape",
        "moe": "SigLIP-so400m-shape + Mixtral-8x7B-shape",
        "long": "SigLIP-so400m-shape + Llama-3.1-8B-shape, 8 images per 65536-token sample",
    }.get(shape, shape)


def build_trainer(args, rank: int, world: int, local_rank: int):
    device = torch.device("cuda", local_rank)
    plan = args.parallelism
    if world == 1:
        return SingleDeviceTrainer(args.shape, args.samples_per_gpu, args.microbatch, device)
    if plan == "ep" or (plan == "auto" and SHAPES[args.shape].moe):
        return ExpertParallelTrainer(args.shape, args.samples_per_gpu, args.microbatch, device, dist.group.WORLD)
    if plan == "cp" or (plan == "auto" and SHAPES[args.shape].images_per_sample > 1):
        return ContextParallelTrainer(args.shape, args.samples_per_gpu, args.microbatch, device, dist.group.WORLD)
    if plan == "tp":
        return TensorParallelTrainer(args.shape, args.samples_per_gpu, args.microbatch, device, dist.group.WORLD)
    if plan == "auto" and world in (2, 4):
        plan = "dp"
    if plan == "dp":
        return SingleDeviceTrainer(args.shape, args.samples_per_gpu, args.microbatch, device, dp_group=dist.group.WORLD)
    from .bench_parallel import PipelineTrainer

    return PipelineTrainer(args, rank, world, device)
