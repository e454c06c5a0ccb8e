"""``utils.tensorboard``: torch's implementation (tensorplay/utils/tensorboard*)."""
from torch.utils.tensorboard import *  # noqa: F401,F403


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
