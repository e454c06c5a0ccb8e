"""``distributed.tensor``: DTensor and placements (torch's implementation) plus the
tensor-parallel styles of this package in ``tensor.parallel``."""
from torch.distributed.tensor import (DTensor, Partial, Placement, Replicate, Shard, distribute_module,  # noqa: F401
                                      distribute_tensor)

from torch.distributed.tensor import (empty, full, init_device_mesh, ones, rand, randn, zeros)  # noqa: F401

from . import experimental, parallel  # noqa: F401


def __getattr__(name):
    """Other DTensor factory and helper names resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.tensor', 'torch.distributed.device_mesh']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
