"""Flight recorder: a ring buffer of the most recent collective / kernel-launch records per
process, dumped as JSON on demand or on failure, and a small analyser that finds the first
sequence number at which ranks disagree (after tensorplay/distributed/flight_recorder
__init__.py:35-108 and its ``fr_trace`` analyser)."""
from __future__ import annotations

import json
import os
import threading
import time
from collections import deque
from typing import Dict, List, Optional

_lock = threading.Lock()
_ring: deque = deque(maxlen=int(os.environ.get("TP_FLIGHT_RECORDER_SIZE", "2048")))
_seq = 0
_enabled = os.environ.get("TP_FLIGHT_RECORDER", "1") != "0"


def record(op: str, **fields) -> int:
    """Append one record; returns its sequence number."""
    global _seq
    if not _enabled:
        return -1
    with _lock:
        _seq += 1
        _ring.append({"seq": _seq, "t": time.time(), "op": op, **fields})
        return _seq


def entries() -> List[dict]:
    with _lock:
        return list(_ring)


def clear() -> None:
    global _seq
    with _lock:
        _ring.clear()
        _seq = 0


def dump(path: Optional[str] = None, rank: Optional[int] = None) -> str:
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    path = path or os.environ.get("TP_FLIGHT_RECORDER_DUMP") or f"flight_recorder_rank{rank}.json"
    if "{rank}" in path:
        path = path.format(rank=rank)
    with open(path, "w") as f:
        json.dump({"rank": rank, "pid": os.getpid(), "entries": entries()}, f)
    return path


def analyze(paths: List[str]) -> Dict:
    """Compare per-rank dumps: first index where the op sequences differ, and ranks that are
    behind (fewer records) - the usual signature of a hang."""
    dumps = [json.load(open(p)) for p in paths]
    seqs = {d["rank"]: [(e["op"], e.get("numel"), e.get("group")) for e in d["entries"]] for d in dumps}
    n = min(len(s) for s in seqs.values()) if seqs else 0
    mismatch = None
    for i in range(n):
        vals = {r: s[i] for r, s in seqs.items()}
        if len(set(vals.values())) > 1:
            mismatch = {"index": i, "per_rank": {r: list(v) for r, v in vals.items()}}
            break
    longest = max((len(s) for s in seqs.values()), default=0)
    behind = sorted(r for r, s in seqs.items() if len(s) < longest)
    return {"ranks": sorted(seqs), "common_prefix": n, "mismatch": mismatch, "behind": behind}


class FlightRecorder:
    """Object form of the module-level recorder (one per process): ``record``, ``entries``, ``dump``,
    ``clear``; usable as a context manager that dumps on an exception."""

    def __init__(self, dump_path: Optional[str] = None):
        self.dump_path = dump_path

    record = staticmethod(record)
    entries = staticmethod(entries)
    clear = staticmethod(clear)

    def dump(self, path: Optional[str] = None) -> str:
        return dump(path or self.dump_path)

    def __enter__(self):
        return self

    def __exit__(self, exc_type, exc, tb):
        if exc_type is not None:
            self.dump()
        return False


_recorder: Optional[FlightRecorder] = None


def start_flight_recorder(dump_path: Optional[str] = None, size: Optional[int] = None) -> FlightRecorder:
    """Enable recording (optionally with a new ring size) and return the process's recorder."""
    global _recorder, _enabled, _ring
    _enabled = True
    if size is not None and size != _ring.maxlen:
        with _lock:
            _ring = deque(_ring, maxlen=int(size))
    _recorder = FlightRecorder(dump_path)
    return _recorder


def dump_flight_recorder(path: Optional[str] = None) -> str:
    return (_recorder or FlightRecorder()).dump(path)


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
