"""``utils.tensorboard``: torch's implementation (tensorplay/utils/tensorboard*)."""
from torch.utils.tensorboard import *  # noqa: F401,F403
