"""Collectives with autograd formulas and RemoteModule (tensorplay/distributed/nn): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.nn as _impl

sys.modules[__name__] = _impl
