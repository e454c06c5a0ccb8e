"""Environment-variable defaults for launcher arguments: PyTorch's module of the same role, under the reference's path."""
import sys

import torch.distributed.argparse_util as _impl

sys.modules[__name__] = _impl
