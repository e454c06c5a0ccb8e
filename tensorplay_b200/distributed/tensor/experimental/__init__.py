"""Experimental DTensor features: context parallelism (ring attention) and implicit replication
(tensorplay/distributed/tensor/experimental/__init__.py, _context_parallel/_attention.py:997-1086)."""
from torch.distributed.tensor.experimental import implicit_replication  # noqa: F401

from ....parallel.cp import (context_parallel, context_parallel_shard, context_parallel_unshard,  # noqa: F401
                             ring_attention)

__all__ = ["context_parallel", "context_parallel_shard", "context_parallel_unshard", "ring_attention",
           "implicit_replication"]
