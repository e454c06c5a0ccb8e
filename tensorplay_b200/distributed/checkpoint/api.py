from __future__ import annotations

import json
import os
import threading
from concurrent.futures import Future
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.distributed as dist

from ... import serialization

META_FILE = ".metadata"


@dataclass
class ShardedTensor:
    """A rank's piece of a global tensor: ``local`` covers ``[offsets, offsets + local.shape)``."""
    local: torch.Tensor
    global_shape: Tuple[int, ...]
    offsets: Tuple[int, ...]


class Stateful:
    """Protocol: objects with ``state_dict()`` / ``load_state_dict()`` are expanded on save/load."""

    def state_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        raise NotImplementedError


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _flatten(sd: Mapping[str, Any], prefix: str = "") -> Dict[str, Any]:
    out = {}
    for k, v in sd.items():
        key = f"{prefix}{k}"
        if hasattr(v, "state_dict") and callable(v.state_dict) and not isinstance(v, torch.Tensor):
            out.update(_flatten(v.state_dict(), key + "."))
        elif isinstance(v, Mapping):
            out.update(_flatten(v, key + "."))
        else:
            out[key] = v
    return out


def _as_sharded(v) -> Optional[ShardedTensor]:
    if isinstance(v, ShardedTensor):
        return v
    try:
        from torch.distributed.tensor import DTensor, Shard
        if isinstance(v, DTensor):
            # offsets from the placement arithmetic itself: two mesh dimensions sharding one tensor
            # dimension, strided shards and uneven / empty trailing shards all come out right
            from torch.distributed.tensor._utils import compute_local_shape_and_global_offset
            shape, offs = compute_local_shape_and_global_offset(v.shape, v.device_mesh, v.placements)
            local = v.to_local()
            if tuple(local.shape) != tuple(shape):   # padded local storage: keep the logical part
                local = local[tuple(slice(0, n) for n in shape)]
            return ShardedTensor(local, tuple(v.shape), tuple(offs))
    except Exception:
        pass
    return None


def _plan_save(flat: Dict[str, Any], rank: int):
    tensors, meta = {}, {}
    for k, v in flat.items():
        st = _as_sharded(v)
        if st is not None:
            tensors[k] = st.local
            meta[k] = {"kind": "sharded", "global_shape": list(st.global_shape), "dtype": str(st.local.dtype),
                       "chunks": [{"rank": rank, "offsets": list(st.offsets), "sizes": list(st.local.shape)}]}
        elif isinstance(v, torch.Tensor):
            if rank == 0:  # replicated tensors are written once
                tensors[k] = v
            meta[k] = {"kind": "replicated", "global_shape": list(v.shape), "dtype": str(v.dtype), "rank": 0}
        else:
            meta[k] = {"kind": "object", "value": v if _jsonable(v) else repr(v)}
    return tensors, meta


def _jsonable(v) -> bool:
    try:
        json.dumps(v)
        return True
    except TypeError:
        return False


def _write(checkpoint_id: str, rank: int, tensors: Dict[str, torch.Tensor], all_meta: Optional[List[dict]],
           wait_for: int = 0, timeout_s: float = 1800.0) -> None:
    """Writes this rank's shard file; the coordinator (``all_meta`` given) writes ``.metadata`` LAST.
    ``wait_for`` > 0 (asynchronous saves, where no collective orders the ranks' background threads):
    every rank drops a ``.done_<rank>`` marker after its shard, and the coordinator waits for that many
    markers before the metadata, so a directory with ``.metadata`` always holds every shard."""
    import time
    os.makedirs(checkpoint_id, exist_ok=True)
    host = {k: t.detach().to("cpu") for k, t in tensors.items()}
    serialization.save_mega(host, os.path.join(checkpoint_id, f"__{rank}_0.distcp"))
    if wait_for:
        with open(os.path.join(checkpoint_id, f".done_{rank}"), "w") as f:
            f.write("1")
    if all_meta is not None:
        if wait_for:
            deadline = time.time() + timeout_s
            names = [os.path.join(checkpoint_id, f".done_{r}") for r in range(wait_for)]
            while not all(os.path.exists(n) for n in names):
                if time.time() > deadline:
                    raise TimeoutError(f"async_save: not every rank finished its shard of {checkpoint_id!r}")
                time.sleep(0.01)
            for n in names:
                os.remove(n)
        merged: Dict[str, dict] = {}
        for m in all_meta:
            for k, e in m.items():
                if k in merged and e["kind"] == "sharded":
                    merged[k]["chunks"].extend(e["chunks"])
                elif k not in merged:
                    merged[k] = e
        tmp = os.path.join(checkpoint_id, META_FILE + ".tmp")
        with open(tmp, "w") as f:
            json.dump({"version": "1.0.0", "world_size": len(all_meta), "state_dict_metadata": merged}, f)
        os.replace(tmp, os.path.join(checkpoint_id, META_FILE))  # the checkpoint is valid once this exists


class MegaStorageWriter:
    """Selects this package's own layout (one ``.mega`` container per rank + ``.metadata``) explicitly:
    ``save(state, storage_writer=MegaStorageWriter(directory))``."""

    def __init__(self, path: str):
        self.path = str(path)


class MegaStorageReader:
    def __init__(self, path: str):
        self.path = str(path)


def save(state_dict: Mapping[str, Any], *, checkpoint_id: Optional[str] = None, process_group=None,
         storage_writer=None, planner=None, **kw) -> None:
    """Collective save of ``state_dict`` (tensors, ``ShardedTensor`` / DTensor shards, Stateful
    objects, plain values) into the directory ``checkpoint_id``. A ``storage_writer`` or ``planner``
    (``FileSystemWriter``, ``DefaultSavePlanner`` ...: PyTorch's planner / storage layer) selects
    PyTorch's implementation and on-disk layout for the whole call."""
    from .hf_storage import HuggingFaceStorageWriter, save_hf
    from .planner import DefaultSavePlanner
    if isinstance(storage_writer, HuggingFaceStorageWriter):
        flat = _flatten(state_dict)
        if any(_as_sharded(v) is not None for v in flat.values()):
            raise ValueError("the Hugging Face layout stores whole tensors: gather sharded entries first "
                             "(get_model_state_dict(..., StateDictOptions(full_state_dict=True))) or consolidate a "
                             "sharded checkpoint with consolidate_to_hf")
        return save_hf({k: v for k, v in flat.items() if isinstance(v, torch.Tensor)}, storage_writer.path,
                       process_group=process_group, fqn_to_file_index=storage_writer.fqn_to_index_mapping)
    if isinstance(storage_writer, MegaStorageWriter):
        checkpoint_id, storage_writer = storage_writer.path, None
    own_planner = planner if isinstance(planner, DefaultSavePlanner) else None
    if storage_writer is not None or (planner is not None and own_planner is None):
        import torch.distributed.checkpoint as tdcp
        return tdcp.save(state_dict, checkpoint_id=checkpoint_id, storage_writer=storage_writer, planner=planner,
                         process_group=process_group, **kw)
    world, rank = _world(process_group)
    flat = _flatten(state_dict)
    pl = own_planner or DefaultSavePlanner()
    local = pl.create_local_plan(rank, flat)
    plans = [local]
    if world > 1:
        plans = [None] * world
        dist.all_gather_object(plans, local, group=process_group)
    final, meta = pl.create_global_plan(plans)    # every rank computes the same global plan
    mine = {it.key for it in final[rank].items if it.kind != "object"}
    tensors = {}
    for k in mine:
        st = _as_sharded(flat[k])
        tensors[k] = st.local if st is not None else flat[k]
    _write(checkpoint_id, rank, tensors, None)
    if world > 1:
        dist.barrier(group=process_group)   # every shard is on disk before the metadata vouches for it
    if rank == 0:
        tmp = os.path.join(checkpoint_id, META_FILE + ".tmp")
        with open(tmp, "w") as f:
            json.dump({"version": "1.0.0", "world_size": world, "state_dict_metadata": meta}, f)
        os.replace(tmp, os.path.join(checkpoint_id, META_FILE))
    if world > 1:
        dist.barrier(group=process_group)


def async_save(state_dict: Mapping[str, Any], *, checkpoint_id: str, process_group=None) -> Future:
    """Stage to host memory now, write in a background thread; the returned future resolves when
    this rank's files are on disk (collectives happen before the function returns). ``.metadata``
    appears only after every rank's shard is complete. Ranks are the ranks of ``process_group``:
    groups that save at the same time need directories of their own."""
    world, rank = _world(process_group)
    tensors, meta = _plan_save(_flatten(state_dict), rank)
    staged = {k: t.detach().to("cpu", copy=True) for k, t in tensors.items()}
    all_meta = [meta]
    if world > 1:
        all_meta = [None] * world
        dist.all_gather_object(all_meta, meta, group=process_group)
    fut: Future = Future()

    # a stale metadata file of an earlier save into this directory must not vouch for new shards
    if rank == 0 and os.path.exists(os.path.join(checkpoint_id, META_FILE)):
        os.remove(os.path.join(checkpoint_id, META_FILE))
    if world > 1:
        dist.barrier(group=process_group)

    def work():
        try:
            _write(checkpoint_id, rank, staged, all_meta if rank == 0 else None, wait_for=world)
            fut.set_result(checkpoint_id)
        except Exception as e:  # pragma: no cover
            fut.set_exception(e)
    threading.Thread(target=work, daemon=True).start()
    return fut


def _overlap(dst_off, dst_size, src_off, src_size):
    lo = [max(a, b) for a, b in zip(dst_off, src_off)]
    hi = [min(a + s, b + t) for a, s, b, t in zip(dst_off, dst_size, src_off, src_size)]
    if any(h <= l for l, h in zip(lo, hi)):
        return None
    return lo, hi


def load(state_dict: Dict[str, Any], *, checkpoint_id: Optional[str] = None, process_group=None,
         storage_reader=None, planner=None, **kw) -> Dict[str, Any]:
    """Fill ``state_dict`` in place from the checkpoint: tensors are overwritten, ``ShardedTensor``
    entries receive the slices that overlap their ``[offsets, offsets + shape)`` window (whatever
    the sharding was at save time), Stateful objects get ``load_state_dict``. With a
    ``storage_reader`` or ``planner`` the call goes to PyTorch's implementation (see :func:`save`)."""
    from .hf_storage import HuggingFaceStorageReader, load_hf
    from .planner import DefaultLoadPlanner
    if isinstance(storage_reader, HuggingFaceStorageReader):
        flat = _flatten(state_dict)
        got = load_hf(storage_reader.path, keys=set(flat))
        for k, v in flat.items():
            st = _as_sharded(v)
            if st is not None:
                st.local.copy_(got[k][tuple(slice(o, o + n) for o, n in zip(st.offsets, st.local.shape))])
            elif isinstance(v, torch.Tensor):
                v.copy_(got[k])
        return state_dict
    if isinstance(storage_reader, MegaStorageReader):
        checkpoint_id, storage_reader = storage_reader.path, None
    if isinstance(planner, DefaultLoadPlanner):
        planner = None
    if storage_reader is not None or planner is not None:
        import torch.distributed.checkpoint as tdcp
        tdcp.load(state_dict, checkpoint_id=checkpoint_id, storage_reader=storage_reader, planner=planner,
                  process_group=process_group, **kw)
        return state_dict
    with open(os.path.join(checkpoint_id, META_FILE)) as f:
        meta = json.load(f)["state_dict_metadata"]
    files: Dict[int, dict] = {}

    def file_of(rank):
        if rank not in files:
            files[rank] = serialization.load_mega(os.path.join(checkpoint_id, f"__{rank}_0.distcp"), mmap=True)
        return files[rank]

    def fill(prefix: str, sd):
        for k in list(sd.keys()):
            v = sd[k]
            key = f"{prefix}{k}"
            if hasattr(v, "state_dict") and callable(v.state_dict) and not isinstance(v, torch.Tensor):
                inner = v.state_dict()
                fill(key + ".", inner)
                v.load_state_dict(inner)
                continue
            if isinstance(v, dict):
                fill(key + ".", v)
                continue
            if key not in meta:
                raise KeyError(f"{key!r} is not in checkpoint {checkpoint_id!r}")
            e = meta[key]
            st = _as_sharded(v)
            if e["kind"] == "object":
                sd[k] = e["value"]
            elif st is not None:
                if e["kind"] == "replicated":
                    src = file_of(e["rank"])[key]
                    sl = tuple(slice(o, o + s) for o, s in zip(st.offsets, st.local.shape))
                    st.local.copy_(src[sl])
                else:
                    for ch in e["chunks"]:
                        ov = _overlap(st.offsets, st.local.shape, ch["offsets"], ch["sizes"])
                        if ov is None:
                            continue
                        lo, hi = ov
                        src = file_of(ch["rank"])[key]
                        ssl = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, ch["offsets"]))
                        dsl = tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, st.offsets))
                        st.local[dsl].copy_(src[ssl])
            elif isinstance(v, torch.Tensor):
                if e["kind"] == "replicated":
                    v.copy_(file_of(e["rank"])[key])
                else:  # saved sharded, wanted whole
                    for ch in e["chunks"]:
                        sl = tuple(slice(o, o + s) for o, s in zip(ch["offsets"], ch["sizes"]))
                        v[sl].copy_(file_of(ch["rank"])[key])
    fill("", state_dict)
    return state_dict


# ------------------------------------------------------------------ sharded-engine glue
def engine_state_dict(engine) -> Dict[str, Any]:
    """Sharded state of a ``FSDPEngine``: per unit the fp32 master weights and Adam moments as
    1-D ``ShardedTensor``s over the unit's (unpadded) flat length, plus the step counter."""
    sd: Dict[str, Any] = {"step": engine.step_count}
    for u in engine.units:
        lo, hi = u.shard_range()
        n = max(0, min(hi, u.numel) - lo)
        for name, t in (("master", u.master), ("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq)):
            sd[f"{u.name}.{name}"] = ShardedTensor(t[:n], (u.numel,), (min(lo, u.numel),))
        if u.local is not None:
            r = engine.rank
            for name, t in (("master", u.local.master), ("exp_avg", u.local.exp_avg), ("exp_avg_sq", u.local.exp_avg_sq)):
                sd[f"{u.name}.experts.rank{r}.{name}"] = ShardedTensor(t[: u.local.numel], (u.local.numel,), (0,))
    return sd


def load_engine_state_dict(engine, checkpoint_id: str) -> None:
    sd = engine_state_dict(engine)
    load(sd, checkpoint_id=checkpoint_id, process_group=engine.group)
    engine.step_count = int(sd["step"])
    # refresh the bf16 parameter shards from the restored masters
    for u in engine.units:
        u.shard.copy_(u.master.to(u.shard.dtype)) if u.shard.numel() == u.master.numel() else None
        if u.local is not None:
            u.local.shard.copy_(u.local.master.to(u.local.shard.dtype))
