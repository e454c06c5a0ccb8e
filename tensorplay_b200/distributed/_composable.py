"""Composable ``replicate`` / ``checkpoint`` / contract registry (tensorplay/distributed/_composable): PyTorch's module of the
same role for those, and this framework's ``fully_shard`` family under ``_composable.fsdp``."""
import sys
import types

import torch.distributed._composable as _impl
from torch.distributed._composable import *  # noqa: F401,F403

from . import fsdp as _fsdp

fsdp = types.ModuleType(__name__ + ".fsdp", "fully_shard and its companions (this framework's implementation).")
for _n in getattr(_fsdp, "__all__", dir(_fsdp)):
    if hasattr(_fsdp, _n):
        setattr(fsdp, _n, getattr(_fsdp, _n))
sys.modules[fsdp.__name__] = fsdp


def __getattr__(name):
    return getattr(_impl, name)


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
