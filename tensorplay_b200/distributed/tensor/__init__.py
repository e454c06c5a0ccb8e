"""``distributed.tensor``: DTensor and placements (torch's implementation) plus the
tensor-parallel styles of this package in ``tensor.parallel``."""
from torch.distributed.tensor import (DTensor, Partial, Placement, Replicate, Shard, distribute_module,  # noqa: F401
                                      distribute_tensor)

from torch.distributed.tensor import (empty, full, init_device_mesh, ones, rand, randn, zeros)  # noqa: F401

from . import experimental, parallel  # noqa: F401

from_local = DTensor.from_local


def linspace(start, end, steps, *, device_mesh=None, placements=None, **kw):
    """``torch.linspace`` distributed over ``device_mesh`` with ``placements`` (replicated by default)."""
    import torch
    return distribute_tensor(torch.linspace(start, end, steps, **kw), device_mesh, placements)


def logspace(start, end, steps, base: float = 10.0, *, device_mesh=None, placements=None, **kw):
    import torch
    return distribute_tensor(torch.logspace(start, end, steps, base=base, **kw), device_mesh, placements)



def __getattr__(name):
    """Other DTensor factory and helper names resolve to PyTorch's."""
    import importlib
    for mod in ['torch.distributed.tensor', 'torch.distributed.device_mesh']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
