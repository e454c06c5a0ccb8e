"""FSDP: ``fully_shard`` (FSDP2-style, per-module sharding with forward/backward hooks) and the
``FullyShardedDataParallel`` wrapper facade.

Two implementations live in this package:

* ``fully_shard`` below is the general, API-compatible path for arbitrary modules: parameters are
  sharded on dim 0 (ceil chunks, padded to the first chunk like the reference,
  tensorplay/distributed/fsdp/_fully_shard/_fsdp_param.py:284-374) into one flat shard per unit, a
  forward pre-hook all-gathers the unit with ONE collective and copies the full parameters out, a
  post-hook frees them, and a backward hook reduce-scatters the unit's gradients with one
  collective into ``param.grad`` shards (plus an all-reduce over the replicate dimension of a 2-D
  mesh). It runs on gloo and NCCL through torch.distributed and is what the CPU oracle uses.
* ``tensorplay_b200.parallel.FSDPEngine`` is the performance path for transformer stacks (flat
  per-layer buffers, peer-memory kernels, optimizer fused into backward).

Knobs follow tensorplay/distributed/fsdp/_fully_shard/_fully_shard.py:66-455 and _fsdp_api.py:20-75.
"""
from __future__ import annotations

from .api import (AllGather, BackwardPrefetch, Comm, CPUOffload, CPUOffloadPolicy, DataParallelMeshDims, FSDPModule,
                  FullyShardedDataParallel, MixedPrecision, MixedPrecisionPolicy, OffloadPolicy, ReduceScatter,
                  ShardingStrategy, UnshardHandle, fully_shard, register_fsdp_forward_method, share_comm_ctx)

from .state_dict_api import (FullOptimStateDictConfig, FullStateDictConfig, LocalOptimStateDictConfig,
                             LocalStateDictConfig, OptimStateDictConfig, ShardedGradScaler, ShardedOptimStateDictConfig,
                             ShardedStateDictConfig, StateDictConfig, StateDictSettings, StateDictType)

__all__ = ["StateDictType", "StateDictConfig", "FullStateDictConfig", "LocalStateDictConfig", "ShardedStateDictConfig",
           "OptimStateDictConfig", "FullOptimStateDictConfig", "LocalOptimStateDictConfig", "ShardedOptimStateDictConfig",
           "StateDictSettings", "ShardedGradScaler", "fully_shard", "DataParallelMeshDims", "FSDPModule", "MixedPrecisionPolicy", "CPUOffloadPolicy", "OffloadPolicy",
           "FullyShardedDataParallel", "ShardingStrategy", "MixedPrecision", "CPUOffload", "BackwardPrefetch",
           "Comm", "AllGather", "ReduceScatter", "UnshardHandle", "register_fsdp_forward_method", "share_comm_ctx"]


def __getattr__(name):
    """``FlatParameter`` and other names without a definition here resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.fsdp', 'torch.distributed.fsdp._flat_param']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
