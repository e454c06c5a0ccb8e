"""Registry of this framework's environment knobs (the reference's counterpart: the ``TP_*`` variables and
``tensorplay/distributed/config.py`` flags). ``flags()`` lists every knob with its current value, default and meaning;
``get(name)`` reads one with its default applied; ``describe()`` is the table as text. The knobs are read where they act
(at arena creation, at library load ...): this module documents and reads them, it is not a second source of truth."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Optional


@dataclass(frozen=True)
class Flag:
    name: str
    default: str
    doc: str

    @property
    def value(self) -> str:
        return os.environ.get(self.name, self.default)

    @property
    def is_set(self) -> bool:
        return self.name in os.environ


_FLAGS = [
    Flag("TPB_DEBUG", "0", "1: load libtpb200_dbg.so, the kernel build whose index guards report the site of an out-of-range "
                           "index through the status word (DeviceIndexError) instead of only skipping the access."),
    Flag("TPB_NO_AUTOBUILD", "0", "1: never compile a missing kernel or runtime library at import; fail with the load error."),
    Flag("TPB_JIT_CACHE", "~/.cache/tensorplay_b200_jit", "Directory of utils.cpp_jit's compiled host extensions."),
    Flag("TPB_SYMM_ALLOC", "vmm", "Symmetric-memory arena: 'vmm' (cuMemCreate + fd export + cuMemMap, NVSwitch multicast "
                                  "mapping) or 'ipc' (cudaMalloc + CUDA-IPC handles, no multicast)."),
    Flag("TPB_SYMM_MULTICAST", "1", "0: do not create the multicast object over the arena (multimem paths fall back to peer loads)."),
    Flag("TPB_SYMM_CANARY", "0", "1: guard bytes behind every arena allocation, checked at close and at exit."),
    Flag("TPB_COMM_TRANSPORT", "ce", "In-step transport of the sharded engine: 'ce' copy engines (default: takes no SM from "
                                     "the GEMMs it overlaps), 'sm' peer-load kernels, 'mc' multicast stores + multimem reduce."),
    Flag("TPB_GATHER_CTAS", "24", "CTAs of the pull all-gather kernel ('sm' transport)."),
    Flag("TPB_REDUCE_CTAS", "148", "CTAs of the reduce-scatter + AdamW kernel."),
    Flag("TPB_REDUCE_OVERLAP", "", "'threads,max_shared': shrink the reduce + AdamW kernel so that it can share SMs with the GEMMs."),
    Flag("TPB_ADAMW_OVERLAP", "", "'ctas_per_sm,max_shared': the same for the single-GPU AdamW on its side stream."),
    Flag("TPB_STORE_BIND_ADDR", "", "Address the TCP store server binds to (the launcher sets 127.0.0.1 for one-node jobs)."),
    Flag("TPB_EVENTS_FILE", "", "File that the 'file' destination of elastic events appends JSON lines to."),
    Flag("TPB_RDZV_EVENTS_DESTINATION", "null", "Destination of rendezvous events: 'null', 'console' or 'file'."),
]
_BY_NAME: Dict[str, Flag] = {f.name: f for f in _FLAGS}


def flags() -> Dict[str, Flag]:
    return dict(_BY_NAME)


def get(name: str) -> str:
    try:
        return _BY_NAME[name].value
    except KeyError:
        raise KeyError(f"{name!r} is not a knob of this framework; known: {sorted(_BY_NAME)}") from None


def get_bool(name: str) -> bool:
    return get(name).strip().lower() not in ("", "0", "false", "no", "off")


def describe(only_set: bool = False) -> str:
    rows = [f for f in _FLAGS if f.is_set or not only_set]
    width = max(len(f.name) for f in rows) if rows else 0
    return "\n".join(f"{f.name:<{width}}  = {f.value!r:<12} (default {f.default!r}): {f.doc}" for f in rows)


def register(name: str, default: str, doc: str) -> Flag:
    """Adds a knob of an extension to the table (same name twice: the definitions must agree)."""
    f = Flag(name, default, doc)
    if name in _BY_NAME and _BY_NAME[name] != f:
        raise ValueError(f"{name} is already registered with another default or description")
    if name not in _BY_NAME:
        _FLAGS.append(f)
        _BY_NAME[name] = f
    return f
