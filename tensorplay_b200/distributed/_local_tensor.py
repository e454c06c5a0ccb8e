"""Single-process simulation of per-rank tensors (tensorplay/distributed/_local_tensor): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed._local_tensor as _impl

sys.modules[__name__] = _impl
