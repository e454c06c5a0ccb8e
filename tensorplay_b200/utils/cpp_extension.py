"""``utils.cpp_extension``: torch's implementation (tensorplay/utils/cpp_extension*)."""
from torch.utils.cpp_extension import *  # noqa: F401,F403
