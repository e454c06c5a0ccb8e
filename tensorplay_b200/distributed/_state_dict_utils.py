"""State-dict gathering / broadcasting helpers: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed._state_dict_utils as _impl

sys.modules[__name__] = _impl
