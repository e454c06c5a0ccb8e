"""Checkpoints in the Hugging Face layout: ``model-0000i-of-0000N.safetensors`` shards plus
``model.safetensors.index.json`` (``weight_map``), written by rank, readable by any safetensors
consumer, and a consolidation step that merges a sharded checkpoint of this package into that
layout (tensorplay/distributed/checkpoint/hf_storage.py: ``HuggingFaceStorageWriter`` / ``Reader``,
``consolidate_safetensors_files``)."""
from __future__ import annotations

import json
import os
from typing import Dict, Mapping, Optional

import torch
import torch.distributed as dist

from ...serialization import load_safetensors, save_safetensors

INDEX = "model.safetensors.index.json"


def _name(i: int, n: int) -> str:
    return f"model-{i + 1:05d}-of-{n:05d}.safetensors"


def save_hf(state_dict: Mapping[str, torch.Tensor], directory: str, *, process_group=None,
            fqn_to_file_index: Optional[Mapping[str, int]] = None) -> None:
    """Collective. Full (unsharded) tensors only: every rank passes the same keys; tensor *k* is
    written by rank ``fqn_to_file_index[k] - 1`` if given, else the tensors are dealt to the ranks by
    size. Rank 0 writes the index."""
    init = dist.is_available() and dist.is_initialized()
    world = dist.get_world_size(process_group) if init else 1
    rank = dist.get_rank(process_group) if init else 0
    os.makedirs(directory, exist_ok=True)
    keys = sorted(state_dict, key=lambda k: -state_dict[k].numel() * state_dict[k].element_size())
    owner: Dict[str, int] = {}
    load = [0] * world
    for k in keys:
        r = (fqn_to_file_index[k] - 1) if fqn_to_file_index is not None else min(range(world), key=lambda q: load[q])
        owner[k] = r
        load[r] += state_dict[k].numel() * state_dict[k].element_size()
    mine = {k: state_dict[k].detach().cpu().contiguous() for k in state_dict if owner[k] == rank}
    save_safetensors(mine, os.path.join(directory, _name(rank, world)), metadata={"format": "pt"})
    if rank == 0:
        total = sum(t.numel() * t.element_size() for t in state_dict.values())
        with open(os.path.join(directory, INDEX), "w") as f:
            json.dump({"metadata": {"total_size": total},
                       "weight_map": {k: _name(owner[k], world) for k in sorted(state_dict)}}, f, indent=2)
    if world > 1:
        dist.barrier(group=process_group)


def load_hf(directory: str, keys=None, map_location=None) -> Dict[str, torch.Tensor]:
    """Reads the tensors named by ``keys`` (all by default) through the index; a directory with a single
    ``model.safetensors`` and no index is accepted too."""
    idx = os.path.join(directory, INDEX)
    if not os.path.exists(idx):
        sd = load_safetensors(os.path.join(directory, "model.safetensors"))
        return {k: (v.to(map_location) if map_location else v) for k, v in sd.items() if keys is None or k in keys}
    with open(idx) as f:
        wm = json.load(f)["weight_map"]
    out: Dict[str, torch.Tensor] = {}
    by_file: Dict[str, list] = {}
    for k, fn in wm.items():
        if keys is None or k in keys:
            by_file.setdefault(fn, []).append(k)
    for fn, ks in by_file.items():
        sd = load_safetensors(os.path.join(directory, fn))
        for k in ks:
            out[k] = sd[k].to(map_location) if map_location else sd[k]
    return out


def consolidate_to_hf(checkpoint_id: str, out_dir: str, max_shard_bytes: int = 5 << 30) -> None:
    """One process: read a sharded checkpoint of this package (``.metadata`` + per-rank files), assemble
    every tensor whole and write it as size-bounded safetensors shards with an index."""
    from .api import META_FILE, ShardedTensor, load
    with open(os.path.join(checkpoint_id, META_FILE)) as f:
        meta = json.load(f)["state_dict_metadata"]
    full: Dict[str, torch.Tensor] = {}
    want = {}
    for k, e in meta.items():
        if e["kind"] == "object":
            continue
        dt = getattr(torch, e["dtype"].split(".")[-1])
        t = torch.zeros(e["global_shape"], dtype=dt)
        want[k] = t if e["kind"] == "replicated" else ShardedTensor(t, tuple(e["global_shape"]), (0,) * t.dim())
        full[k] = t
    load(want, checkpoint_id=checkpoint_id)
    os.makedirs(out_dir, exist_ok=True)
    groups, cur, size = [], {}, 0
    for k in sorted(full):
        nb = full[k].numel() * full[k].element_size()
        if cur and size + nb > max_shard_bytes:
            groups.append(cur)
            cur, size = {}, 0
        cur[k] = full[k]
        size += nb
    if cur:
        groups.append(cur)
    wm = {}
    for i, g in enumerate(groups):
        save_safetensors(g, os.path.join(out_dir, _name(i, len(groups))), metadata={"format": "pt"})
        for k in g:
            wm[k] = _name(i, len(groups))
    with open(os.path.join(out_dir, INDEX), "w") as f:
        json.dump({"metadata": {"total_size": sum(t.numel() * t.element_size() for t in full.values())},
                   "weight_map": wm}, f, indent=2)


class HuggingFaceStorageWriter:
    """``save(state, storage_writer=HuggingFaceStorageWriter(dir))`` writes the HF layout."""

    def __init__(self, path: str, fqn_to_index_mapping: Optional[Mapping[str, int]] = None):
        self.path, self.fqn_to_index_mapping = str(path), fqn_to_index_mapping


class HuggingFaceStorageReader:
    def __init__(self, path: str):
        self.path = str(path)
