"""``distributed.fsdp._fully_shard``: the reference's private path of ``fully_shard`` and its companions. The names of this
framework's implementation (``fsdp/api.py``) are shown here; the internals of PyTorch's implementation (``_fsdp_param``,
``_fsdp_collectives`` ...) stay importable as PyTorch's modules of those paths."""
from .. import api as _api
from ..api import *  # noqa: F401,F403

__all__ = [n for n in ("CPUOffloadPolicy", "FSDPModule", "MixedPrecisionPolicy", "OffloadPolicy", "UnshardHandle",
                       "fully_shard", "register_fsdp_forward_method", "share_comm_ctx", "Comm", "AllGather", "ReduceScatter",
                       "DataParallelMeshDims", "get_cls_to_fsdp_cls") if hasattr(_api, n)]


def __getattr__(name):
    import importlib
    if hasattr(_api, name):
        return getattr(_api, name)
    for mod in ("torch.distributed.fsdp._fully_shard", "torch.distributed.fsdp._fully_shard._fully_shard",
                "torch.distributed.fsdp._fully_shard._fsdp_api", "torch.distributed.fsdp._fully_shard._fsdp_common"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
