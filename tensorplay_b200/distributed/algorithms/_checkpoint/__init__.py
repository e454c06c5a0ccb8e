"""Module wrappers for activation checkpointing and offload (tensorplay/distributed/algorithms/_checkpoint): PyTorch's
``checkpoint_wrapper`` module under the reference's package path - the wrappers act on any ``nn.Module`` and recompute
through autograd, which the custom autograd functions of this framework support. The sharded engine of this framework
has its own per-block policies (``FSDPEngine(activation_checkpointing=...)``)."""
from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import (ActivationWrapper, CheckpointImpl,  # noqa: F401
                                                                         CheckpointWrapper, OffloadWrapper,
                                                                         apply_activation_checkpointing,
                                                                         checkpoint_wrapper, offload_wrapper)

__all__ = ["ActivationWrapper", "CheckpointImpl", "CheckpointWrapper", "OffloadWrapper", "apply_activation_checkpointing",
           "checkpoint_wrapper", "offload_wrapper"]
