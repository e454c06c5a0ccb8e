"""Import path of the checkpointable-tensor protocol (tensorplay/distributed/checkpoint/protocol.py)."""
from . import CheckpointableTensor  # noqa: F401


def _is_checkpointable_tensor(obj) -> bool:
    import torch
    return isinstance(obj, torch.Tensor) and isinstance(obj, CheckpointableTensor)
