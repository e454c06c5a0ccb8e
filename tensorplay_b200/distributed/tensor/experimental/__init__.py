"""Experimental DTensor features: context parallelism (ring attention) and implicit replication
(tensorplay/distributed/tensor/experimental/__init__.py, _context_parallel/_attention.py:997-1086)."""
from torch.distributed.tensor.experimental import implicit_replication  # noqa: F401

from ....parallel.cp import (context_parallel, context_parallel_shard, context_parallel_unshard,  # noqa: F401
                             ring_attention)

__all__ = ["context_parallel", "context_parallel_shard", "context_parallel_unshard", "ring_attention",
           "implicit_replication"]


def __getattr__(name):
    """``local_map``, ``register_sharding`` and other experimental DTensor helpers resolve to PyTorch's."""
    import importlib
    for mod in ("torch.distributed.tensor.experimental", "torch.distributed.tensor.experimental._attention"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
