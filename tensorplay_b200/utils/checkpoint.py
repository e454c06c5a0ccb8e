"""Activation checkpointing (torch's reentrant-free implementation; API as in
tensorplay/utils/checkpoint.py:210-547). The sharded engine has its own per-unit checkpointing
that also re-gathers parameters (``tensorplay_b200.parallel.engine``)."""
from torch.utils.checkpoint import (CheckpointPolicy, checkpoint, checkpoint_sequential,  # noqa: F401
                                    create_selective_checkpoint_contexts)

__all__ = ["checkpoint", "checkpoint_sequential", "CheckpointPolicy", "create_selective_checkpoint_contexts"]


def __getattr__(name):
    """The remaining names of the activation-checkpoint module resolve to PyTorch's."""
    import importlib
    for mod in ['torch.utils.checkpoint']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
