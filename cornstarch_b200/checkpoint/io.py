"""State-dict files in the HF layout: safetensors (or torch ``.bin``) shards plus an index JSON.

Index schema (identical to HF / the reference's ``CheckpointIndexFile``):
``{"metadata": {"total_size": <bytes>}, "weight_map": {<param name>: <file name>}}``.
File naming follows the reference's sharded writer
(cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_checkpoint_io.py:244-287):
``model-00001.safetensors`` for a single writer, ``model-stage-000NN-shard-000MM.safetensors`` when a
pipeline stage writes its own shards.
"""

from __future__ import annotations

import json
import os
from typing import Iterable

import torch

SAFE_INDEX = "model.safetensors.index.json"
BIN_INDEX = "pytorch_model.bin.index.json"
SAFE_SINGLE = "model.safetensors"
BIN_SINGLE = "pytorch_model.bin"


def _nbytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


def _save_file(sd: dict[str, torch.Tensor], path: str, use_safetensors: bool) -> None:
    if use_safetensors:
        from safetensors.torch import save_file

        save_file({k: v.contiguous() for k, v in sd.items()}, path, metadata={"format": "pt"})
    else:
        torch.save(sd, path)


def _load_file(path: str) -> dict[str, torch.Tensor]:
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file

        return load_file(path)
    return torch.load(path, map_location="cpu", weights_only=True)


def shard_state_dict(sd: dict[str, torch.Tensor], max_shard_size: int | None) -> list[dict[str, torch.Tensor]]:
    """Greedy split in insertion order so that no shard exceeds ``max_shard_size`` bytes (one tensor may)."""
    if not max_shard_size:
        return [sd]
    shards, cur, cur_size = [], {}, 0
    for k, v in sd.items():
        n = _nbytes(v)
        if cur and cur_size + n > max_shard_size:
            shards.append(cur)
            cur, cur_size = {}, 0
        cur[k] = v
        cur_size += n
    if cur:
        shards.append(cur)
    return shards


def save_state_dict_sharded(sd: dict[str, torch.Tensor], directory: str, max_shard_size: int | None = None,
                            use_safetensors: bool = True, stage: int | None = None, base: str = "model",
                            write_index: bool = True) -> dict:
    """Write ``sd`` under ``directory``; returns the index dict.  ``max_shard_size`` in bytes (None = one file)."""
    os.makedirs(directory, exist_ok=True)
    ext = ".safetensors" if use_safetensors else ".bin"
    if base == "model" and not use_safetensors:
        base = "pytorch_model"
    shards = shard_state_dict(sd, max_shard_size)
    index = {"metadata": {"total_size": sum(_nbytes(v) for v in sd.values())}, "weight_map": {}}
    single = len(shards) == 1 and stage is None and max_shard_size is None
    for i, shard in enumerate(shards):
        if single:
            fname = (SAFE_SINGLE if use_safetensors else BIN_SINGLE) if base in ("model", "pytorch_model") else base + ext
        elif stage is None:
            fname = f"{base}-{i + 1:05d}{ext}"
        else:
            fname = f"{base}-stage-{stage + 1:05d}-shard-{i + 1:05d}{ext}"
        _save_file(shard, os.path.join(directory, fname), use_safetensors)
        for k in shard:
            index["weight_map"][k] = fname
    if write_index and not single:
        with open(os.path.join(directory, SAFE_INDEX if use_safetensors else BIN_INDEX), "w") as f:
            json.dump(index, f, indent=2, sort_keys=True)
    return index


def merge_indices(indices: Iterable[dict]) -> dict:
    """Union of per-stage indices (sizes summed, weight maps merged)."""
    out = {"metadata": {"total_size": 0}, "weight_map": {}}
    for idx in indices:
        out["metadata"]["total_size"] += idx["metadata"]["total_size"]
        out["weight_map"].update(idx["weight_map"])
    return out


def find_index(path: str) -> str | None:
    for name in (SAFE_INDEX, BIN_INDEX):
        p = os.path.join(path, name)
        if os.path.isfile(p):
            return p
    return None


def load_state_dict_any(path: str, wanted: set[str] | None = None) -> dict[str, torch.Tensor]:
    """Load from a directory (index or single file) or a single file path; ``wanted`` limits which shard files are read."""
    if os.path.isfile(path):
        sd = _load_file(path)
        return sd if wanted is None else {k: v for k, v in sd.items() if k in wanted}
    idx_path = find_index(path)
    if idx_path is not None:
        with open(idx_path) as f:
            index = json.load(f)
        files = sorted({fn for k, fn in index["weight_map"].items() if wanted is None or k in wanted})
        out = {}
        for fn in files:
            part = _load_file(os.path.join(path, fn))
            out.update(part if wanted is None else {k: v for k, v in part.items() if k in wanted})
        return out
    for name in (SAFE_SINGLE, BIN_SINGLE):
        p = os.path.join(path, name)
        if os.path.isfile(p):
            sd = _load_file(p)
            return sd if wanted is None else {k: v for k, v in sd.items() if k in wanted}
    raise FileNotFoundError(f"no checkpoint found under {path}")
