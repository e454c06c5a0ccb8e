"""Helper functions of the distributed wrappers (tensorplay/distributed/utils.py): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.utils as _impl

sys.modules[__name__] = _impl
