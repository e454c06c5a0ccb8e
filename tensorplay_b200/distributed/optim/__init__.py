"""Distributed optimizers: ``ZeroRedundancyOptimizer`` (ZeRO stage 1, ``zero.py``). The sharded training
engine and the fused DDP path of this package shard optimizer state natively as well."""
from .zero import ZeroRedundancyOptimizer  # noqa: F401


def __getattr__(name):
    """Functional / post-local-SGD / named optimizers resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.optim']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
