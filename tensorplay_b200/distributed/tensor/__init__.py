"""``distributed.tensor``: DTensor and placements (torch's implementation) plus the
tensor-parallel styles of this package in ``tensor.parallel``."""
from torch.distributed.tensor import (DTensor, Partial, Placement, Replicate, Shard, distribute_module,  # noqa: F401
                                      distribute_tensor)

from torch.distributed.tensor import (empty, full, init_device_mesh, ones, rand, randn, zeros)  # noqa: F401

from . import experimental, parallel  # noqa: F401
