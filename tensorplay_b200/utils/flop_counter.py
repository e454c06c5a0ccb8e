"""``utils.flop_counter``: torch's implementation (tensorplay/utils/flop_counter*)."""
from torch.utils.flop_counter import *  # noqa: F401,F403
