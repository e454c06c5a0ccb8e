"""Default timeouts of the process groups: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.constants as _impl

sys.modules[__name__] = _impl
