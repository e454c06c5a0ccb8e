"""Distributed optimizers: ``ZeroRedundancyOptimizer`` (ZeRO-1; torch's implementation). The
sharded training engine and the fused DDP path of this package shard optimizer state natively."""
from torch.distributed.optim import ZeroRedundancyOptimizer  # noqa: F401
