"""Fused AdamW over flat parameter / gradient / state buffers ("arena"), with optional ZeRO-1 sharding.

On CUDA with bf16 parameters the optimizer re-homes every parameter into one contiguous bf16 buffer per
weight-decay group (in module order, so q/k/v and gate/up weights end up adjacent and can run as one
GEMM), gives every parameter a ``main_grad`` view into a flat gradient buffer (the linear / norm /
embedding backward kernels accumulate straight into it) and keeps fp32 master weights and Adam moments
flat as well.  One kernel launch per group then does: unscale / clip, Adam moments, decoupled weight
decay, master update, bf16 write-back and gradient zeroing.  The global gradient norm is a reduction
kernel plus a 1-thread kernel that turns it into the clip factor on the device, so a step has no host
synchronisation.

With ``zero_stage=1`` and a data-parallel group each rank keeps the master weights and moments of its
1/dp slice only: gradients are reduce-scattered (or all-reduced by the caller), the slice is updated, the
bf16 parameters are all-gathered.

On CPU (or non-bf16 parameters) the same math runs in PyTorch on ordinary ``.grad`` tensors; this is
the oracle of the GPU test and the path of the CPU/gloo tests.

Stands in for ``torch.optim.Adam(fused=True)`` plus ColossalAI's ``HybridParallelAMPOptimizer`` /
``HybridParallelNaiveOptimizer`` (master weights, gradient clipping across tp/pp, dynamic loss scale),
used at cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:627-654.
"""

from __future__ import annotations

import os
from typing import Iterable

import torch
import torch.distributed as dist

from ..ops import _native as nat

ALIGN = 64  # elements; keeps every parameter 128-byte aligned inside the arena


class _Region:
    """One weight-decay group laid out flat."""

    def __init__(self, params: list[torch.nn.Parameter], grad_dtype: torch.dtype, shard: tuple[int, int] | None,
                 grad_alloc=None, split_master: bool = False):
        dev = params[0].device
        self.params = params
        self.offsets = []
        n = 0
        for p in params:
            self.offsets.append(n)
            n += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        ws = shard[1] if shard else 1
        pad_to = ALIGN * ws
        self.numel = (n + pad_to - 1) // pad_to * pad_to
        self.flat_param = torch.zeros(self.numel, dtype=torch.bfloat16, device=dev)
        # gradients may live in peer-mapped memory so that the data-parallel reduction kernel can reach them
        self.flat_grad = grad_alloc(self.numel) if grad_alloc is not None else torch.zeros(self.numel, dtype=grad_dtype, device=dev)
        for p, off in zip(params, self.offsets):
            view = self.flat_param[off : off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.flat_grad[off : off + p.numel()].view(p.shape)
            p.grad_added_to_main_grad = False
        if shard:
            r, ws = shard
            per = self.numel // ws
            self.lo, self.hi = r * per, (r + 1) * per
        else:
            self.lo, self.hi = 0, self.numel
        k = self.hi - self.lo
        # fp32 master weights, or (split_master) only their lower 16 bits: the bf16 parameter is the upper half, so
        # master bits = (parameter bits << 16) + remainder and 2 bytes per parameter are saved
        self.split_master = split_master
        if split_master:
            self.master = None
            self.resid = torch.zeros(k, dtype=torch.int16, device=dev)
        else:
            self.master = self.flat_param[self.lo : self.hi].float()
            self.resid = None
        self.exp_avg = torch.zeros(k, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(k, dtype=torch.float32, device=dev)

    def master_weights(self) -> torch.Tensor:
        """The fp32 master weights of this rank's slice (a new tensor when they are stored split)."""
        if not self.split_master:
            return self.master
        hi = self.flat_param[self.lo : self.hi].view(torch.int16).to(torch.int32) << 16
        return (hi + self.resid.to(torch.int32)).view(torch.float32)

    def set_master_weights(self, sl: slice, master: torch.Tensor) -> None:
        """Write fp32 master weights for ``sl`` of this rank's slice (and, stored split, the bf16 parameters they imply)."""
        master = master.reshape(-1).to(device=self.flat_param.device, dtype=torch.float32)
        if not self.split_master:
            self.master[sl].copy_(master)
            return
        bits = master.view(torch.int32)
        hi = (bits + 0x8000) >> 16  # round half away from zero; as int32 its low 16 bits are the bf16 pattern
        self.resid[sl].copy_((bits - (hi << 16)).to(torch.int16))
        self.flat_param[self.lo : self.hi][sl].view(torch.int16).copy_(hi.to(torch.int16))

    def gathered_states(self, group=None) -> dict[str, torch.Tensor]:
        """``master`` / ``exp_avg`` / ``exp_avg_sq`` over the WHOLE region (length ``numel``).  When the region is sharded
        over ``group`` (ZeRO-1) the slices of all ranks are all-gathered: a collective call."""
        local = {"master": self.master_weights(), "exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq}
        if self.hi - self.lo == self.numel:
            return local
        assert group is not None, "a sharded region needs its data-parallel group to assemble the full state"
        out = {}
        for k, v in local.items():
            full = torch.empty(self.numel, dtype=torch.float32, device=v.device)
            dist.all_gather_into_tensor(full, v.contiguous(), group=group)
            out[k] = full
        return out

    def import_param_state(self, off: int, numel: int, st: dict) -> None:
        """Copy the part of one parameter's (whole) state that falls into this rank's slice."""
        lo, hi = max(off, self.lo), min(off + numel, self.hi)
        if lo >= hi:
            return
        src, dst = slice(lo - off, hi - off), slice(lo - self.lo, hi - self.lo)
        self.set_master_weights(dst, st["master"].reshape(-1)[src])
        self.exp_avg[dst].copy_(st["exp_avg"].reshape(-1)[src])
        self.exp_avg_sq[dst].copy_(st["exp_avg_sq"].reshape(-1)[src])

    def reset_master_weights(self) -> None:
        """Master weights := the current bf16 parameters."""
        if self.split_master:
            self.resid.zero_()
        else:
            self.master.copy_(self.flat_param[self.lo : self.hi].float())


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_norm: float = 0.0, grad_dtype: torch.dtype = torch.bfloat16,
                 zero_stage: int = 0, dp_group=None, norm_groups: list | None = None, use_arena: bool | None = None,
                 expert_group=None, fused_dp: bool = True, split_master: bool | None = None):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)
        # split_master: keep only the lower 16 bits of each fp32 master weight next to the bf16 parameter (which is its
        # upper half): the same fp32 update with 2 bytes per parameter less.  Default on; CORNSTARCH_B200_FP32_MASTER=1
        # (or split_master=False) stores whole fp32 master weights.
        self.split_master = (os.environ.get("CORNSTARCH_B200_FP32_MASTER", "0") != "1") if split_master is None else split_master
        self.max_norm = max_norm
        self.grad_dtype = grad_dtype
        self.zero_stage = zero_stage
        self.dp_group = dp_group
        self.norm_groups = norm_groups or []  # extra groups (tp, pp) over which the squared norm is summed
        # param groups flagged {"expert_parallel": True} hold parameters that are NOT replicated over the data-parallel
        # group (each rank owns different experts): never ZeRO-sharded; their squared norm is summed over expert_group
        self.expert_group = expert_group
        self.fused_dp = fused_dp  # reduce data-parallel gradients with this package's peer-memory kernel when possible
        self.reducer = None
        self.loss_scale = 1.0
        self._step = 0
        self._regions: list[tuple[dict, _Region]] = []
        all_params = [p for g in self.param_groups for p in g["params"]]
        cuda_bf16 = bool(all_params) and all(p.is_cuda and p.dtype == torch.bfloat16 for p in all_params)
        self.use_arena = cuda_bf16 if use_arena is None else (use_arena and cuda_bf16)
        if self.use_arena:
            self._build_arena()

    # ------------------------------------------------------------------ arena path
    def _build_arena(self):
        self._overlap, self._overlap_used = None, False
        shard = None
        if self.zero_stage >= 1 and self.dp_group is not None and dist.get_world_size(self.dp_group) > 1:
            shard = (dist.get_rank(self.dp_group), dist.get_world_size(self.dp_group))
        if self.fused_dp and self.dp_group is not None and self.grad_dtype == torch.bfloat16:
            from ..parallel.dp_fused import FusedGradReducer

            self.reducer = FusedGradReducer.get(self.dp_group)
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.requires_grad]
            if ps:
                alloc = self.reducer.allocate if (self.reducer is not None and not g.get("expert_parallel")) else None
                region = _Region(ps, self.grad_dtype, None if g.get("expert_parallel") else shard, alloc,
                                 split_master=self.split_master)
                region.sharded = shard is not None and not g.get("expert_parallel")
                region.expert = bool(g.get("expert_parallel"))
                self._regions.append((g, region))
        dev = self._regions[0][1].flat_param.device
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        # block sums of the norm kernel, added in block order so that replicas with equal gradients get equal norms
        self._sumsq_scratch = torch.zeros(4096, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)
        self._sumsq_expert = torch.zeros(1, dtype=torch.float32, device=dev)
        self._sharded = shard is not None

    def flat_grads(self) -> list[torch.Tensor]:
        """The flat gradient buffers of replicated parameters (what data-parallel reduction works on)."""
        return [r.flat_grad for _, r in self._regions if not r.expert]

    def overlapped_reduce(self, max_ctas: int = 16):
        """Context manager for the forward + backward pass of a step's LAST micro-batch: the gradients of each decoder
        layer are averaged over the data-parallel group while the backward pass of the earlier layers still runs;
        ``reduce_dp_grads()`` afterwards reduces the rest and closes the exchange.  A null context when the peer-memory
        reducer is not in use (single rank, NCCL path, ZeRO-1)."""
        import contextlib

        if (not self.use_arena or self.reducer is None or self._sharded or self.dp_group is None
                or dist.get_world_size(self.dp_group) == 1):
            return contextlib.nullcontext()
        from ..parallel.dp_fused import OverlappedGradReduce

        if self._overlap is None:
            self._overlap = OverlappedGradReduce(self.reducer, self.flat_grads(), max_ctas)
        self._overlap_used = True
        return self._overlap

    def reduce_dp_grads(self, bucket_bytes: int = 256 << 20) -> bool:
        """Average the replicated gradients over the data-parallel group.  Returns False when there is nothing to do
        here (no group, ZeRO-1 reduces inside ``step``, or the plain per-parameter path is in use)."""
        if not self.use_arena or self.dp_group is None or dist.get_world_size(self.dp_group) == 1 or self._sharded:
            return False
        # gradients that autograd left in ``.grad`` (embedding lookups, norm weights behind a tensor-parallel reduction,
        # sliced views, PyTorch fallbacks) must be part of what is averaged: fold them in before anything is reduced
        folded = self._fold_stray_grads()
        bufs = self.flat_grads()
        if self.reducer is not None:
            if self._overlap is not None and self._overlap_used:
                # part of the buffers was reduced during the backward pass; a range that a fold touched afterwards
                # holds mean + local remainder and is averaged once more (the mean of that is the full mean)
                self._overlap.finish(redo=self._spans_in_flat_grads(folded, bufs))
                self._overlap_used = False
            else:
                self.reducer.reduce(bufs)
            return True
        for flat in bufs:
            step = max(1, bucket_bytes // flat.element_size())
            for s in range(0, flat.numel(), step):
                dist.all_reduce(flat[s : s + step], op=dist.ReduceOp.AVG, group=self.dp_group)
        return True

    def flat_params(self) -> list[torch.Tensor]:
        return [r.flat_param for _, r in self._regions]

    def _fold_stray_grads(self) -> list:
        """Gradients autograd left in ``.grad`` (ops without main_grad fusion) are added to ``main_grad``.  Returns the
        parameters that had one.  A parameter that had a stray gradient once is reported on every later call too, so
        that all data-parallel ranks agree on the set even when one of them happens to see no gradient in a step."""
        sticky = self.__dict__.setdefault("_stray_params", {})
        for _, r in self._regions:
            for p in r.params:
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                    p.grad = None
                    sticky[id(p)] = p
        return list(sticky.values())

    @staticmethod
    def _spans_in_flat_grads(params: list, bufs: list[torch.Tensor]) -> list[tuple[int, int, int]]:
        """``(buffer index, lo, hi)`` element ranges (64-element aligned, as the arena lays parameters out) of the
        ``main_grad`` views of ``params`` inside the flat gradient buffers ``bufs``."""
        out = []
        for p in params:
            g = p.main_grad
            for bi, flat in enumerate(bufs):
                off = (g.data_ptr() - flat.data_ptr()) // flat.element_size()
                if g.data_ptr() >= flat.data_ptr() and off < flat.numel():
                    out.append((bi, off // ALIGN * ALIGN, min(flat.numel(), (off + g.numel() + ALIGN - 1) // ALIGN * ALIGN)))
                    break
        return sorted(out)

    def _reduce_partial_grads(self):
        """Parameters whose gradient is a partial sum on every rank of a group (norm weights under token-sharded tensor
        parallelism carry ``tp_partial_grad_group``): add the parts, once per step."""
        for g in self.param_groups:
            for p in g["params"]:
                grp = getattr(p, "tp_partial_grad_group", None)
                if grp is None or dist.get_world_size(grp) < 2:
                    continue
                t = p.main_grad if self.use_arena else p.grad
                if t is not None:
                    dist.all_reduce(t, group=grp)

    def _step_arena(self):
        lib = nat.lib()
        st = nat.stream()
        self._fold_stray_grads()
        self._reduce_partial_grads()
        if self.dp_group is not None and dist.get_world_size(self.dp_group) > 1:
            # expert gradients hold the contributions of every data-parallel rank's tokens, each taken from that
            # rank's own mean loss: the mean over ranks is 1/dp of the sum
            for _, r in self._regions:
                if r.expert:
                    r.flat_grad.mul_(1.0 / dist.get_world_size(self.dp_group))
        if self._sharded and not getattr(self, "grads_already_reduced", False):
            todo = [r for _, r in self._regions if r.sharded]
            if self.reducer is not None and todo:
                # reduce-scatter by the peer-memory kernel: every rank ends up with the mean of its own slice
                self.reducer.reduce([r.flat_grad for r in todo], all_reduce=False)
            else:
                for r in todo:
                    out = r.flat_grad[r.lo : r.hi]
                    dist.reduce_scatter_tensor(out, r.flat_grad, op=dist.ReduceOp.AVG, group=self.dp_group)
        inv_scale = 1.0 / self.loss_scale
        # kernels with bounded waits (peer-memory reductions, fused TP / CP / EP) report a wait that ran out in the
        # device's status word; the update is then skipped on the device, and the host learns of it without a sync
        gate = nat.status_word(self._sumsq.device) if nat.status_in_use(self._sumsq.device) else None
        need_norm = self.max_norm > 0 or self.loss_scale != 1.0 or gate is not None
        if need_norm:
            self._sumsq.zero_()
            self._sumsq_expert.zero_()
            any_expert = False
            for _, r in self._regions:
                g = r.flat_grad[r.lo : r.hi]
                acc = self._sumsq_expert if r.expert else self._sumsq
                any_expert |= r.expert
                nat.check(lib.csb_sumsq(g.data_ptr(), int(g.dtype == torch.float32), g.numel(), acc.data_ptr(),
                                        self._sumsq_scratch.data_ptr(), self._sumsq_scratch.numel(), st), "csb_sumsq")
            if self._sharded and dist.get_world_size(self.dp_group) > 1:
                dist.all_reduce(self._sumsq, group=self.dp_group)  # every rank summed its slice only
            if any_expert:
                if self.expert_group is not None and dist.get_world_size(self.expert_group) > 1:
                    dist.all_reduce(self._sumsq_expert, group=self.expert_group)
                self._sumsq.add_(self._sumsq_expert)
            for grp in self.norm_groups:
                if grp is not None and dist.get_world_size(grp) > 1:
                    dist.all_reduce(self._sumsq, group=grp)
            nat.check(lib.csb_clip_scale(self._sumsq.data_ptr(), float(self.max_norm), inv_scale, self._scale.data_ptr(),
                                         self._norm.data_ptr(), self._skip.data_ptr(), nat.ptr(gate), st), "csb_clip_scale")
            nat.poll_status(self._sumsq.device)
        self._step += 1
        for g, r in self._regions:
            b1, b2 = g["betas"]
            bc1 = 1.0 - b1 ** self._step
            bc2 = 1.0 - b2 ** self._step
            grad = r.flat_grad[r.lo : r.hi]
            param = r.flat_param[r.lo : r.hi]
            step_fn = lib.csb_adamw_split if r.split_master else lib.csb_adamw
            nat.check(
                step_fn(param.data_ptr(), (r.resid if r.split_master else r.master).data_ptr(), r.exp_avg.data_ptr(), r.exp_avg_sq.data_ptr(),
                              grad.data_ptr(), int(grad.dtype == torch.float32), grad.numel(), float(g["lr"]), b1, b2,
                              float(g["eps"]), float(g["weight_decay"]), bc1, bc2,
                              self._scale.data_ptr() if need_norm else None, self._skip.data_ptr() if need_norm else None,
                              1, st),
                "csb_adamw",
            )
            if r.sharded:
                if r.lo > 0:
                    r.flat_grad[: r.lo].zero_()
                if r.hi < r.numel:
                    r.flat_grad[r.hi :].zero_()
                dist.all_gather_into_tensor(r.flat_param, param.clone(), group=self.dp_group)
            for p in r.params:
                p.grad_added_to_main_grad = False

    # ------------------------------------------------------------------ plain path (CPU / fp32)
    @torch.no_grad()
    def _step_plain(self):
        self._reduce_partial_grads()
        params = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        inv_scale = 1.0 / self.loss_scale
        scale = inv_scale
        if self.max_norm > 0 or self.loss_scale != 1.0:
            sq = torch.zeros((), dtype=torch.float32, device=params[0].device if params else "cpu")
            sq_expert = torch.zeros_like(sq)
            for p in params:
                if getattr(p, "expert_parallel", False):
                    sq_expert = sq_expert + p.grad.float().pow(2).sum()
                else:
                    sq = sq + p.grad.float().pow(2).sum()
            if self.expert_group is not None and dist.get_world_size(self.expert_group) > 1:
                dist.all_reduce(sq_expert, group=self.expert_group)  # every rank owns different experts
            sq = sq + sq_expert
            for grp in self.norm_groups:
                if grp is not None and dist.get_world_size(grp) > 1:
                    dist.all_reduce(sq, group=grp)
            norm = sq.sqrt() * inv_scale
            self._last_norm = norm
            if not torch.isfinite(norm):
                return
            if self.max_norm > 0:
                scale = inv_scale * min(1.0, self.max_norm / (float(norm) + 1e-6))
        self._step += 1
        for g in self.param_groups:
            b1, b2 = g["betas"]
            bc1, bc2 = 1.0 - b1 ** self._step, 1.0 - b2 ** self._step
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["master"] = p.detach().float().clone()
                    st["exp_avg"] = torch.zeros_like(st["master"])
                    st["exp_avg_sq"] = torch.zeros_like(st["master"])
                gr = p.grad.float() * scale
                st["exp_avg"].mul_(b1).add_(gr, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(gr, gr, value=1 - b2)
                denom = (st["exp_avg_sq"] / bc2).sqrt().add_(g["eps"])
                st["master"].mul_(1 - g["lr"] * g["weight_decay"]).addcdiv_(st["exp_avg"] / bc1, denom, value=-g["lr"])
                p.copy_(st["master"].to(p.dtype))

    @torch.no_grad()
    def step(self, closure=None):
        from ..utils.trace import nvtx_range

        with nvtx_range("optimizer/fused_adamw_step"):
            return self._step_impl(closure)

    def _step_impl(self, closure=None):
        loss = closure() if closure is not None else None
        if self.use_arena:
            self._step_arena()
        else:
            self._step_plain()
        return loss

    def zero_grad(self, set_to_none: bool = True):
        if self.use_arena:
            # the fused step already cleared the flat gradient buffer; only stray .grad tensors remain
            for _, r in self._regions:
                for p in r.params:
                    p.grad = None
            return
        super().zero_grad(set_to_none)

    def clear_main_grads(self):
        for _, r in self._regions:
            r.flat_grad.zero_()

    def grad_norm(self) -> torch.Tensor | None:
        """Global gradient norm of the last step (device scalar; reading it synchronises)."""
        if self.use_arena:
            return self._norm
        return getattr(self, "_last_norm", None)

    # ------------------------------------------------------------------ state dict in the per-parameter layout
    def state_dict(self):
        if not self.use_arena:
            sd = super().state_dict()
            sd["fused_step"] = self._step
            return sd
        # expose flat state as per-parameter tensors (ids follow param_groups order, like torch)
        state, idx = {}, 0
        index_of = {}
        for g in self.param_groups:
            for p in g["params"]:
                index_of[id(p)] = idx
                idx += 1
        # ZeRO-1: every rank assembles the whole state (a collective over the data-parallel group), so that the file a
        # single rank writes is complete and parameters that straddle a slice boundary are whole
        for _, r in self._regions:
            full = r.gathered_states(self.dp_group)
            for p, off in zip(r.params, r.offsets):
                s = slice(off, off + p.numel())
                state[index_of[id(p)]] = {k: v[s].view(p.shape).clone() for k, v in full.items()}
        groups = []
        start = 0
        for g in self.param_groups:
            d = {k: v for k, v in g.items() if k != "params"}
            d["params"] = list(range(start, start + len(g["params"])))
            start += len(g["params"])
            groups.append(d)
        return {"state": state, "param_groups": groups, "fused_step": self._step}

    def load_state_dict(self, sd):
        self._step = int(sd.get("fused_step", 0))
        if not self.use_arena:
            sd = {k: v for k, v in sd.items() if k != "fused_step"}
            return super().load_state_dict(sd)
        index_of, idx = {}, 0
        for g in self.param_groups:
            for p in g["params"]:
                index_of[id(p)] = idx
                idx += 1
        for g, saved in zip(self.param_groups, sd["param_groups"]):
            for k, v in saved.items():
                if k != "params":
                    g[k] = v
        for _, r in self._regions:
            for p, off in zip(r.params, r.offsets):
                st = sd["state"].get(index_of[id(p)])
                if st is None:
                    continue
                r.import_param_state(off, p.numel(), st)

    def update_master_params(self):
        """Re-read master weights from the (just loaded) bf16 parameters."""
        for _, r in self._regions:
            r.reset_master_weights()


def split_decay_groups(model: torch.nn.Module, weight_decay: float = 0.01) -> list[dict]:
    """Two param groups in module order: matrices (decayed) and vectors (norm weights, biases; not decayed)."""
    decay, no_decay, expert, seen = [], [], [], set()
    for p in model.parameters():
        if not p.requires_grad or id(p) in seen:
            continue
        seen.add(id(p))
        if getattr(p, "expert_parallel", False):
            expert.append(p)  # sharded over an expert-parallel group: its own region, never ZeRO-sharded or DP-reduced
        else:
            (decay if p.dim() >= 2 else no_decay).append(p)
    groups = []
    if decay:
        groups.append({"params": decay, "weight_decay": weight_decay})
    if no_decay:
        groups.append({"params": no_decay, "weight_decay": 0.0})
    if expert:
        groups.append({"params": expert, "weight_decay": weight_decay, "expert_parallel": True})
    return groups
