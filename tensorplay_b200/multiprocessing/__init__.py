"""``multiprocessing``: ``spawn`` / ``start_processes`` / ``ProcessContext`` and shared-memory tensor
passing (torch.multiprocessing; API as in tensorplay/multiprocessing/spawn.py:80-283)."""
from torch.multiprocessing import *  # noqa: F401,F403
from torch.multiprocessing import ProcessContext, get_context, spawn, start_processes  # noqa: F401

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("_fdsharer",))
