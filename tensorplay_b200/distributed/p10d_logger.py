"""Collective-call logger with process-group context (tensorplay/distributed/p10d_logger.py): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.c10d_logger as _impl

sys.modules[__name__] = _impl
