"""`worker/device` descriptors: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.remote_device as _impl

sys.modules[__name__] = _impl
