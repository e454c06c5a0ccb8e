"""``distributed``: process groups and collectives (torch.distributed over gloo / NCCL for the
plumbing), stores, device meshes, DDP, FSDP, pipeline and tensor parallelism, expert parallelism,
distributed checkpointing, the elastic launcher and observability - the surface of
tensorplay/distributed (distributed_core.py:24-104 lists the collective API; names coincide).

The fused compute+collective kernels live in ``tensorplay_b200.parallel``; the wrappers here
route to them on CUDA and to plain collectives on CPU ranks.
"""
from __future__ import annotations

import torch.distributed as _td
from torch.distributed import *  # noqa: F401,F403
from torch.distributed import (Backend, GroupMember, P2POp, ProcessGroup, ReduceOp, Work, all_gather,  # noqa: F401
                               all_gather_into_tensor, all_gather_object, all_reduce, all_to_all,
                               all_to_all_single, barrier, batch_isend_irecv, broadcast,
                               broadcast_object_list, destroy_process_group, gather, get_backend,
                               get_rank, get_world_size, init_process_group, irecv, is_available,
                               is_initialized, isend, monitored_barrier, new_group, recv, reduce,
                               reduce_scatter, reduce_scatter_tensor, scatter, send)

from . import store  # noqa: F401
from .store import FileStore, HashStore, PrefixStore, StoreTimeoutError, TCPStore  # noqa: F401

# reference spellings of the single-tensor collectives
all_gather_single = all_gather_into_tensor
reduce_scatter_single = reduce_scatter_tensor

from ._collective_extras import (SHRINK_ABORT, SHRINK_DEFAULT, AllgatherOptions, all_gather_single_coalesced,  # noqa: E402,F401
                                 gather_into_tensor, gather_single, record_comm, reduce_scatter_coalesced,
                                 reduce_scatter_single_coalesced, register_device_backend, set_timeout)

_LAZY = {"ddp", "fsdp", "device_mesh", "pipelining", "tensor", "checkpoint", "elastic", "run", "launcher",
         "flight_recorder", "watchdog", "_symmetric_memory", "_token_switch", "algorithms", "optim",
         "rendezvous", "debug", "_tools", "rpc", "nn", "utils", "_functional_collectives", "_composable",
         "_composable_state", "_shard", "_local_tensor", "_state_dict_utils", "_checkpointable", "_serialization",
         "collective_utils", "argparse_util", "constants", "remote_device", "logging_handlers", "p10d_logger",
         "_watchdog", "_store", "_tensor", "distributed_core", "_mesh_layout", "_pycute", "config", "autograd"}
# the star import above also copied torch's sub-modules of these names; ours must win
for _n in _LAZY:
    globals().pop(_n, None)
del _n


def __getattr__(name):
    import importlib
    if name in _LAZY:
        return importlib.import_module(f"{__name__}.{name}")
    if name in ("DeviceMesh", "init_device_mesh"):
        from . import device_mesh
        return getattr(device_mesh, name)
    if name in ("default_pg_timeout", "default_pg_nccl_timeout"):
        from torch.distributed import constants
        return getattr(constants, name)
    return getattr(_td, name)
