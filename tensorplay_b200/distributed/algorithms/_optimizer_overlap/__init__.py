"""Optimizer step overlapped with gradient communication for PyTorch's DDP / FSDP classes
(tensorplay/distributed/algorithms/_optimizer_overlap): PyTorch's module. This framework's own wrappers fuse the optimizer
into the reduction instead (``DistributedDataParallel(fused_adamw=...)``, ``FSDPEngine``)."""
from torch.distributed.algorithms._optimizer_overlap.optimizer_overlap import (OverlappedOptimizer, _as_overlapped_optim,  # noqa: F401
                                                                               register_overlapped)

OptimizerOverlap = OverlappedOptimizer     # the reference's name of the base class
as_overlapped_optim = _as_overlapped_optim

__all__ = ["OptimizerOverlap", "OverlappedOptimizer", "as_overlapped_optim", "register_overlapped"]
