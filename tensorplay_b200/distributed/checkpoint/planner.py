"""Save / load planning for distributed checkpoints.

A *save plan* says which rank writes which tensor: sharded entries are written by their owners;
replicated tensors, which every rank holds, are written ONCE, spread over the ranks by size so that
no rank writes everything (the reference's ``DefaultSavePlanner`` de-duplicates the same way,
tensorplay/distributed/checkpoint/default_planner.py: ``dedup_save_plans``). A *load plan* lists,
for every destination window, the saved chunks that overlap it (resharding on load).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass
class WriteItem:
    key: str
    kind: str                       # "sharded" | "replicated" | "object"
    global_shape: Tuple[int, ...] = ()
    offsets: Tuple[int, ...] = ()
    sizes: Tuple[int, ...] = ()
    dtype: str = ""
    nbytes: int = 0
    value: Any = None               # objects only


@dataclass
class SavePlan:
    rank: int
    items: List[WriteItem] = field(default_factory=list)


@dataclass
class ReadItem:
    key: str
    src_rank: int
    src_slices: Tuple[slice, ...]
    dst_slices: Tuple[slice, ...]


def overlap(dst_off, dst_size, src_off, src_size) -> Optional[Tuple[List[int], List[int]]]:
    lo = [max(a, b) for a, b in zip(dst_off, src_off)]
    hi = [min(a + s, b + t) for a, s, b, t in zip(dst_off, dst_size, src_off, src_size)]
    if any(h <= l for l, h in zip(lo, hi)):
        return None
    return lo, hi


class DefaultSavePlanner:
    """``dedup_replicated``: write every replicated tensor once (balanced over the ranks) instead of
    on rank 0 only; ``flatten_state_dict`` is always on (nested dicts and Stateful objects)."""

    def __init__(self, dedup_replicated: bool = True):
        self.dedup_replicated = dedup_replicated

    def create_local_plan(self, rank: int, entries: Dict[str, Any]) -> SavePlan:
        from .api import _as_sharded, _jsonable
        import torch
        plan = SavePlan(rank)
        for k, v in entries.items():
            st = _as_sharded(v)
            if st is not None:
                plan.items.append(WriteItem(k, "sharded", tuple(st.global_shape), tuple(st.offsets), tuple(st.local.shape),
                                            str(st.local.dtype), st.local.numel() * st.local.element_size()))
            elif isinstance(v, torch.Tensor):
                plan.items.append(WriteItem(k, "replicated", tuple(v.shape), (0,) * v.dim(), tuple(v.shape), str(v.dtype),
                                            v.numel() * v.element_size()))
            else:
                plan.items.append(WriteItem(k, "object", value=v if _jsonable(v) else repr(v)))
        return plan

    def create_global_plan(self, plans: List[SavePlan]) -> Tuple[List[SavePlan], Dict[str, dict]]:
        """Returns the per-rank plans after de-duplication and the checkpoint metadata."""
        world = len(plans)
        meta: Dict[str, dict] = {}
        load = [sum(i.nbytes for i in p.items if i.kind == "sharded") for p in plans]
        owner: Dict[str, int] = {}
        replicated = sorted({i.key: i for p in plans for i in p.items if i.kind == "replicated"}.values(),
                            key=lambda i: -i.nbytes)
        for it in replicated:   # largest first onto the least loaded rank
            r = min(range(world), key=lambda q: load[q]) if self.dedup_replicated else 0
            owner[it.key] = r
            load[r] += it.nbytes
        out = []
        for p in plans:
            kept = []
            for it in p.items:
                if it.kind == "sharded":
                    e = meta.setdefault(it.key, {"kind": "sharded", "global_shape": list(it.global_shape),
                                                 "dtype": it.dtype, "chunks": []})
                    e["chunks"].append({"rank": p.rank, "offsets": list(it.offsets), "sizes": list(it.sizes)})
                    kept.append(it)
                elif it.kind == "replicated":
                    meta.setdefault(it.key, {"kind": "replicated", "global_shape": list(it.global_shape),
                                             "dtype": it.dtype, "rank": owner[it.key]})
                    if owner[it.key] == p.rank:
                        kept.append(it)
                else:
                    meta.setdefault(it.key, {"kind": "object", "value": it.value})
            out.append(SavePlan(p.rank, kept))
        return out, meta


class DefaultLoadPlanner:
    """Which saved chunks fill a destination window ``[offsets, offsets + sizes)`` of ``key``."""

    def create_read_items(self, key: str, entry: dict, offsets, sizes) -> List[ReadItem]:
        if entry["kind"] == "replicated":
            sl = tuple(slice(o, o + s) for o, s in zip(offsets, sizes))
            return [ReadItem(key, entry["rank"], sl, tuple(slice(0, s) for s in sizes))]
        items = []
        for ch in entry["chunks"]:
            ov = overlap(offsets, sizes, ch["offsets"], ch["sizes"])
            if ov is None:
                continue
            lo, hi = ov
            items.append(ReadItem(key, ch["rank"],
                                  tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, ch["offsets"])),
                                  tuple(slice(l - o, h - o) for l, h, o in zip(lo, hi, offsets))))
        return items
