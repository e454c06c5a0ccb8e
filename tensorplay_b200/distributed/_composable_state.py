"""Per-module composable state registry: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed._composable_state as _impl

sys.modules[__name__] = _impl
