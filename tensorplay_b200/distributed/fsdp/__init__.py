"""FSDP: ``fully_shard`` (FSDP2-style, per-module sharding with forward/backward hooks) and the
``FullyShardedDataParallel`` wrapper facade.

Two implementations live in this package:

* ``fully_shard`` below is the general, API-compatible path for arbitrary modules: parameters are
  sharded on dim 0 (ceil chunks, padded to the first chunk like the reference,
  tensorplay/distributed/fsdp/_fully_shard/_fsdp_param.py:284-374), a forward pre-hook all-gathers
  a unit's parameters, a post-hook frees them, and a backward hook re-gathers, then
  reduce-scatters gradients into ``param.grad`` shards. It runs on gloo and NCCL through
  torch.distributed and is what the CPU oracle configuration uses.
* ``tensorplay_b200.parallel.FSDPEngine`` is the performance path for transformer stacks (flat
  per-layer buffers, peer-memory kernels, optimizer fused into backward).

Knobs follow tensorplay/distributed/fsdp/_fully_shard/_fully_shard.py:66-455 and _fsdp_api.py:20-75.
"""
from __future__ import annotations

from .api import (BackwardPrefetch, CPUOffload, CPUOffloadPolicy, FSDPModule, FullyShardedDataParallel,
                  MixedPrecision, MixedPrecisionPolicy, OffloadPolicy, ShardingStrategy, fully_shard)

import dataclasses as _dc
from typing import Optional as _Optional


@_dc.dataclass
class DataParallelMeshDims:
    """Names of the mesh dimensions used for sharding and (hybrid) replication."""
    shard: _Optional[str] = None
    replicate: _Optional[str] = None


__all__ = ["fully_shard", "DataParallelMeshDims", "FSDPModule", "MixedPrecisionPolicy", "CPUOffloadPolicy", "OffloadPolicy",
           "FullyShardedDataParallel", "ShardingStrategy", "MixedPrecision", "CPUOffload", "BackwardPrefetch"]


def __getattr__(name):
    """State-dict configuration classes, ``StateDictType``, ``FlatParameter``, ``UnshardHandle`` and ``register_fsdp_forward_method`` resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.fsdp', 'torch.distributed.fsdp._flat_param']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
