"""``utils``: activation checkpointing, data loading (``DistributedSampler``), pytree, hooks."""
from torch.utils import *  # noqa: F401,F403
from torch.utils import _pytree, hooks  # noqa: F401

from . import checkpoint, data  # noqa: F401

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("_dispatch",))
