"""HF-compatible sharded checkpoints under DP x TP x PP, one directory per modality module.

Layout (same tree as the reference, cornstarch/plugin/multimodal_parallel_plugin/
multimodal_parallel_checkpoint_io.py:583-599)::

    <ckpt>/<key>_encoder/module/      config.json, model-stage-000NN-shard-000MM.safetensors, model.safetensors.index.json
    <ckpt>/<key>_encoder/projector/   same (written by the encoder's last stage)
    <ckpt>/language_model/            same
    <optim ckpt>/<modal name>/        optimizer state shards per stage + index + param groups

Rules: only data-parallel rank 0 writes; tensor-parallel shards are gathered to full, un-padded
tensors under their HF names and written by tp rank 0; every pipeline stage writes its own shard
files plus a per-stage index under ``tmp_index_files/``; after a barrier the modality's first stage
merges the indices (sizes summed, weight maps unioned) and writes ``config.json``.  Modules whose
parameters are all frozen are not saved.  ``save_unsharded_model`` is not supported, as in the reference.
Loading reads only the shard files that contain parameters held by this rank and re-shards them.
"""

from __future__ import annotations

import json
import os
import shutil

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import nn as cnn
from ..checkpoint import io as ckio
from ..multimodal.modeling import ModalModuleBase
from ..optim.fused_adamw import FusedAdamW

TMP_INDEX_DIR = "tmp_index_files"


# ---------------------------------------------------------------------------------------------- TP helpers
def _tp_info(module: nn.Module) -> dict[str, tuple]:
    """param name -> (kind, owning module) for tensor-parallel parameters of ``module``."""
    info = {}
    for name, mod in module.named_modules():
        pre = name + "." if name else ""
        if isinstance(mod, cnn.ColumnParallelLinear):
            info[pre + "weight"] = ("col", mod)
            if mod.bias is not None:
                info[pre + "bias"] = ("col", mod)
        elif isinstance(mod, cnn.RowParallelLinear):
            info[pre + "weight"] = ("row", mod)
        elif isinstance(mod, cnn.VocabParallelEmbedding):
            info[pre + "weight"] = ("vocab", mod)
        elif getattr(mod, "parallel", None) == "col" and hasattr(mod, "nx"):  # GPT-2 Conv1D, weight stored [in, out]
            info[pre + "weight"] = ("col_t", mod)
            info[pre + "bias"] = ("col", mod)
        elif getattr(mod, "parallel", None) == "row" and hasattr(mod, "nx"):
            info[pre + "weight"] = ("row_t", mod)
    return info


def _gather(t: torch.Tensor, group) -> list[torch.Tensor]:
    ws = dist.get_world_size(group)
    parts = [torch.empty_like(t) for _ in range(ws)]
    dist.all_gather(parts, t.contiguous(), group=group)
    return parts


def gather_full_tensor(name: str, t: torch.Tensor, info: dict, tp_group) -> torch.Tensor:
    """Full, un-padded tensor of a (possibly tensor-parallel) parameter or optimizer state."""
    if name not in info or tp_group is None or dist.get_world_size(tp_group) == 1:
        return t
    kind, mod = info[name]
    parts = _gather(t, tp_group)
    if kind == "col_t":
        return cnn.unshard_rows([p.t() for p in parts], getattr(mod, "split_sizes", None)).t().contiguous()
    if kind == "row_t":
        return torch.cat(parts, dim=0)
    if kind == "col":
        full = cnn.unshard_rows(parts, getattr(mod, "split_sizes", None))
        v = getattr(mod, "full_vocab_size", None)
        return full[:v] if v is not None else full
    if kind == "row":
        return torch.cat(parts, dim=1)
    full = torch.cat(parts, dim=0)
    return full[: mod.full_num_embeddings]


def shard_full_tensor(name: str, full: torch.Tensor, info: dict, tp_group) -> torch.Tensor:
    if name not in info or tp_group is None or dist.get_world_size(tp_group) == 1:
        return full
    kind, mod = info[name]
    tp, r = dist.get_world_size(tp_group), dist.get_rank(tp_group)
    if kind == "col_t":
        return cnn.shard_rows(full.t(), tp, r, getattr(mod, "split_sizes", None)).t().contiguous()
    if kind == "row_t":
        return full.chunk(tp, dim=0)[r]
    if kind == "col":
        v = getattr(mod, "full_vocab_size", None)
        if v is not None:
            local = mod.weight.shape[0]
            pad = local * tp - full.shape[0]
            if pad > 0:
                full = torch.cat([full, full.new_zeros(pad, *full.shape[1:])], dim=0)
            return full[r * local : (r + 1) * local]
        return cnn.shard_rows(full, tp, r, getattr(mod, "split_sizes", None))
    if kind == "row":
        return full.chunk(tp, dim=1)[r]
    pad = mod.padded_num_embeddings - full.shape[0]
    if pad > 0:
        full = torch.cat([full, full.new_zeros(pad, *full.shape[1:])], dim=0)
    return full[mod.vocab_start : mod.vocab_end]


def _expert_state_keys(model: nn.Module) -> list[str]:
    """State-dict keys (global expert indices) of the parameters that expert parallelism shards over the data-parallel
    group: every rank of that group holds different ones."""
    ptrs = {p.data_ptr() for p in model.parameters() if getattr(p, "expert_parallel", False)}
    if not ptrs:
        return []
    return [k for k, t in model.state_dict().items() if t.data_ptr() in ptrs]


def _checkpoint_param_names(model: nn.Module) -> dict[int, str]:
    """``id(parameter) -> name in the checkpoint``: the module path, except for expert-parallel parameters, whose
    checkpoint name carries the expert's global index (``state_dict`` renames them, ``named_parameters`` does not)."""
    names = {id(p): n for n, p in model.named_parameters()}
    experts = {p.data_ptr(): p for p in model.parameters() if getattr(p, "expert_parallel", False)}
    if experts:
        for k, t in model.state_dict().items():
            p = experts.get(t.data_ptr())
            if p is not None:
                names[id(p)] = k
    return names


class ModalParallelCheckpointIO:
    """Checkpoint IO of one modality's module on the groups that shard it."""

    def __init__(self, dp_group, tp_group, pp_group, stage_manager=None):
        self.dp_group, self.tp_group, self.pp_group = dp_group, tp_group, pp_group
        self.dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
        self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        self.stage_manager = stage_manager
        self.stage = stage_manager.stage_in_modal if stage_manager is not None else 0

    def _barrier(self):
        if self.pp_group is not None:
            dist.barrier(self.pp_group)

    # ---- model
    def save_sharded_model(self, model: nn.Module, path: str, size_per_shard: int = 1024, use_safetensors: bool = True,
                           merge_on_first: bool = True) -> None:
        trainable = any(p.requires_grad for p in model.parameters())
        has_params = any(True for _ in model.parameters())
        info = _tp_info(model)
        sd = {}
        if has_params and trainable:
            for name, t in model.state_dict().items():
                # tensor-parallel gathers are collective over the tp group: every tp rank takes part
                sd[name] = gather_full_tensor(name, t.detach(), info, self.tp_group).cpu().contiguous()
        writer = self.dp_rank == 0 and self.tp_rank == 0
        expert_keys = _expert_state_keys(model)
        if writer and sd:
            os.makedirs(path, exist_ok=True)
            os.makedirs(os.path.join(path, TMP_INDEX_DIR), exist_ok=True)
            index = ckio.save_state_dict_sharded(sd, path, max_shard_size=size_per_shard * 1024 * 1024,
                                                 use_safetensors=use_safetensors, stage=self.stage, write_index=False)
            with open(os.path.join(path, TMP_INDEX_DIR, f"index-stage-{self.stage:05d}.json"), "w") as f:
                json.dump(index, f)
        elif expert_keys and sd and self.tp_rank == 0:
            # expert parallelism: the other data-parallel ranks hold other experts; each writes its own (global names)
            os.makedirs(os.path.join(path, TMP_INDEX_DIR), exist_ok=True)
            index = ckio.save_state_dict_sharded({k: sd[k] for k in expert_keys}, path, max_shard_size=size_per_shard * 1024 * 1024,
                                                 use_safetensors=use_safetensors, stage=self.stage,
                                                 base=f"model-experts-{self.dp_rank:03d}", write_index=False)
            with open(os.path.join(path, TMP_INDEX_DIR, f"index-stage-{self.stage:05d}-experts-{self.dp_rank:03d}.json"), "w") as f:
                json.dump(index, f)
        if merge_on_first:
            if expert_keys and self.dp_group is not None:
                dist.barrier(self.dp_group)  # the merge below reads what every expert writer left
            self._barrier()
            first = self.stage_manager is None or self.stage_manager.is_first_stage(check_only_in_modal=True)
            tmp = os.path.join(path, TMP_INDEX_DIR)
            if writer and first and os.path.isdir(tmp):
                merged = ckio.merge_indices(json.load(open(os.path.join(tmp, f))) for f in sorted(os.listdir(tmp)))
                name = ckio.SAFE_INDEX if use_safetensors else ckio.BIN_INDEX
                with open(os.path.join(path, name), "w") as f:
                    json.dump(merged, f, indent=2, sort_keys=True)
                if hasattr(model, "config") and hasattr(model.config, "save_pretrained"):
                    model.config.save_pretrained(path)
                shutil.rmtree(tmp, ignore_errors=True)
            self._barrier()

    def save_unsharded_model(self, *a, **k):
        raise NotImplementedError("unsharded checkpoints are not supported under pipeline parallelism; use shard=True")

    def load_sharded_model(self, model: nn.Module, path: str, strict: bool = False) -> tuple[list, list]:
        info = _tp_info(model)
        own = model.state_dict()
        loaded = ckio.load_state_dict_any(path, wanted=set(own.keys()))
        missing = [k for k in own if k not in loaded]
        with torch.no_grad():
            for k, full in loaded.items():
                t = shard_full_tensor(k, full, info, self.tp_group)
                own[k].copy_(t.to(own[k].dtype))
        if strict and missing:
            raise RuntimeError(f"missing keys when loading {path}: {missing}")
        return missing, []

    # ---- optimizer
    def save_sharded_optimizer(self, optimizer, model: nn.Module, path: str, size_per_shard: int = 1024) -> None:
        opt = optimizer.unwrap() if hasattr(optimizer, "unwrap") else optimizer
        info = _tp_info(model)
        names = _checkpoint_param_names(model)
        expert_ids = {id(p) for p in model.parameters() if getattr(p, "expert_parallel", False)}
        expert_flat = {}
        sd = opt.state_dict()
        flat = {}
        idx = 0
        for g in opt.param_groups:
            for p in g["params"]:
                st = sd["state"].get(idx)
                n = names.get(id(p))
                if st is not None and n is not None:
                    for k, v in st.items():
                        if isinstance(v, torch.Tensor) and v.dim() > 0 and v.shape == p.shape:
                            v = gather_full_tensor(n, v, info, self.tp_group)
                        flat[f"{n}::{k}"] = v.detach().cpu() if isinstance(v, torch.Tensor) else torch.tensor(v)
                        if id(p) in expert_ids:
                            expert_flat[f"{n}::{k}"] = flat[f"{n}::{k}"]
                idx += 1
        if self.dp_rank != 0 and self.tp_rank == 0 and expert_flat:
            # expert parallelism: the state of the experts this data-parallel rank owns, in files of its own
            os.makedirs(path, exist_ok=True)
            ckio.save_state_dict_sharded(expert_flat, path, max_shard_size=size_per_shard * 1024 * 1024, use_safetensors=False,
                                         base=f"pytorch_optim-stage-{self.stage + 1:05d}-experts-{self.dp_rank:03d}",
                                         write_index=False)
        if self.dp_rank == 0 and self.tp_rank == 0:
            os.makedirs(path, exist_ok=True)
            ckio.save_state_dict_sharded(flat, path, max_shard_size=size_per_shard * 1024 * 1024, use_safetensors=False,
                                         stage=self.stage, base="pytorch_optim", write_index=False)
            groups = [{k: v for k, v in g.items() if k != "params"} for g in sd["param_groups"]]
            torch.save({"param_groups": groups, "fused_step": sd.get("fused_step", 0)},
                       os.path.join(path, f"pytorch_optim_group-stage-{self.stage + 1:05d}.bin"))
        self._barrier()

    def load_sharded_optimizer(self, optimizer, model: nn.Module, path: str) -> None:
        opt = optimizer.unwrap() if hasattr(optimizer, "unwrap") else optimizer
        info = _tp_info(model)
        names = _checkpoint_param_names(model)
        flat = {}
        for fn in sorted(os.listdir(path)):
            if fn.startswith("pytorch_optim-stage-") and fn.endswith(".bin"):
                flat.update(torch.load(os.path.join(path, fn), map_location="cpu", weights_only=True))
        gfile = os.path.join(path, f"pytorch_optim_group-stage-{self.stage + 1:05d}.bin")
        if not os.path.isfile(gfile):
            # written by a pipeline with fewer stages: the hyper-parameters are the same in every stage's file
            others = sorted(fn for fn in os.listdir(path) if fn.startswith("pytorch_optim_group-stage-"))
            if others:
                gfile = os.path.join(path, others[0])
        meta = torch.load(gfile, weights_only=False) if os.path.isfile(gfile) else {"param_groups": [], "fused_step": 0}
        state, idx = {}, 0
        for g in opt.param_groups:
            for p in g["params"]:
                n = names.get(id(p))
                ent = {}
                for key, v in flat.items():
                    pn, _, k = key.partition("::")
                    if pn == n:
                        if v.dim() > 0 and n in info:
                            v = shard_full_tensor(n, v, info, self.tp_group)
                        ent[k] = v.to(p.device) if v.dim() > 0 else v
                if ent:
                    state[idx] = ent
                idx += 1
        groups = []
        start = 0
        for g, saved in zip(opt.param_groups, meta["param_groups"] or [{} for _ in opt.param_groups]):
            d = dict(saved)
            d["params"] = list(range(start, start + len(g["params"])))
            start += len(g["params"])
            groups.append(d)
        if isinstance(opt, FusedAdamW):
            opt.load_state_dict({"state": state, "param_groups": groups, "fused_step": meta.get("fused_step", 0)})
        else:
            cur = opt.state_dict()
            full_groups = []
            for cg, ng in zip(cur["param_groups"], groups):
                merged = dict(cg)
                merged.update({k: v for k, v in ng.items() if k != "params"})
                full_groups.append(merged)
            opt.load_state_dict({"state": state, "param_groups": full_groups})


class MultimodalParallelCheckpointIO:
    """Dispatches to :class:`ModalParallelCheckpointIO` for the modality this rank runs."""

    def __init__(self, plugin):
        self.plugin = plugin

    def _modal_io(self, model) -> ModalParallelCheckpointIO:
        pl = self.plugin
        pp = pl.pp_groups[0] if pl.pp_groups else None
        return ModalParallelCheckpointIO(pl.dp_group, model.tp_group, pp, pl.stage_manager)

    def _world_barrier(self):
        dist.barrier()

    def save_model(self, model, checkpoint: str, shard: bool = True, size_per_shard: int = 1024, use_safetensors: bool = True):
        if not shard:
            raise NotImplementedError("unsharded checkpoints are not supported under pipeline parallelism; use shard=True")
        name = model.my_modal_name
        module = getattr(model.module, name)
        io = self._modal_io(model)
        base = os.path.join(checkpoint, name)
        if isinstance(module, ModalModuleBase):
            io.save_sharded_model(module.module, os.path.join(base, "module"), size_per_shard, use_safetensors, merge_on_first=False)
            if module.projector is not None:
                # the projector lives on one stage only: a plain single-writer save
                pio = ModalParallelCheckpointIO(io.dp_group, io.tp_group, None, None)
                pio.save_sharded_model(module.projector, os.path.join(base, "projector"), size_per_shard, use_safetensors)
            self._world_barrier()
            self._merge(module.module, os.path.join(base, "module"), io, use_safetensors)
        else:
            io.save_sharded_model(module, base, size_per_shard, use_safetensors, merge_on_first=False)
            self._world_barrier()
            self._merge(module, base, io, use_safetensors)
        self._world_barrier()

    @staticmethod
    def _merge(module, path, io: ModalParallelCheckpointIO, use_safetensors):
        first = io.stage_manager is None or io.stage_manager.is_first_stage(check_only_in_modal=True)
        tmp = os.path.join(path, TMP_INDEX_DIR)
        if io.dp_rank == 0 and io.tp_rank == 0 and first and os.path.isdir(tmp):
            merged = ckio.merge_indices(json.load(open(os.path.join(tmp, f))) for f in sorted(os.listdir(tmp)))
            with open(os.path.join(path, ckio.SAFE_INDEX if use_safetensors else ckio.BIN_INDEX), "w") as f:
                json.dump(merged, f, indent=2, sort_keys=True)
            if hasattr(module, "config") and hasattr(module.config, "save_pretrained"):
                module.config.save_pretrained(path)
            shutil.rmtree(tmp, ignore_errors=True)

    def load_model(self, model, checkpoint, strict: bool = False):
        """``checkpoint``: a root directory written by ``save_model`` or a dict
        ``{"language_model": path, "<key>_encoder.module": path, "<key>_encoder.projector": path}``."""
        name = model.my_modal_name
        module = getattr(model.module, name)
        io = self._modal_io(model)

        def resolve(sub: str):
            if isinstance(checkpoint, dict):
                return checkpoint.get(sub)
            p = os.path.join(checkpoint, *sub.split("."))
            return p if os.path.exists(p) else None

        if isinstance(module, ModalModuleBase):
            p = resolve(f"{name}.module")
            if p is not None:
                io.load_sharded_model(module.module, p, strict)
            p = resolve(f"{name}.projector")
            if p is not None and module.projector is not None:
                io.load_sharded_model(module.projector, p, strict)
        else:
            p = resolve(name)
            if p is not None:
                io.load_sharded_model(module, p, strict)
        if model.optimizer is not None and hasattr(model.optimizer, "update_master_params"):
            model.optimizer.update_master_params()
        self._world_barrier()
        return model

    def save_optimizer(self, optimizer, checkpoint: str, shard: bool = True, size_per_shard: int = 1024):
        model = optimizer.model
        io = self._modal_io(model)
        module = getattr(model.module, model.my_modal_name)
        io.save_sharded_optimizer(optimizer, module, os.path.join(checkpoint, model.my_modal_name), size_per_shard)
        self._world_barrier()

    def load_optimizer(self, optimizer, checkpoint: str):
        model = optimizer.model
        io = self._modal_io(model)
        module = getattr(model.module, model.my_modal_name)
        io.load_sharded_optimizer(optimizer, module, os.path.join(checkpoint, model.my_modal_name))
        self._world_barrier()
