"""Distributed optimizers: ``ZeroRedundancyOptimizer`` (ZeRO-1; torch's implementation). The
sharded training engine and the fused DDP path of this package shard optimizer state natively."""
from torch.distributed.optim import ZeroRedundancyOptimizer  # noqa: F401


def __getattr__(name):
    """Functional / post-local-SGD / RPC-based optimizers resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.optim']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
