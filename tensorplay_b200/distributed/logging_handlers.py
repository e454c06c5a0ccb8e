"""Log handler registry of the distributed loggers: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.logging_handlers as _impl

sys.modules[__name__] = _impl
