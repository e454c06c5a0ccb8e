"""Composable `replicate` / `checkpoint` / contract registry (tensorplay/distributed/_composable): PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed._composable as _impl

sys.modules[__name__] = _impl
