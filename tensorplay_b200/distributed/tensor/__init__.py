"""``distributed.tensor``: DTensor and placements (torch's implementation) plus the
tensor-parallel styles of this package in ``tensor.parallel``."""
from torch.distributed.tensor import (DTensor, Partial, Placement, Replicate, Shard, distribute_module,  # noqa: F401
                                      distribute_tensor)

from . import parallel  # noqa: F401
