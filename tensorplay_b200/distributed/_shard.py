"""Legacy ShardedTensor API (tensorplay/distributed/_shard): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed._shard as _impl

sys.modules[__name__] = _impl
