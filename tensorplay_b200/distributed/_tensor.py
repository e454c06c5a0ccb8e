"""``distributed._tensor``: older spelling of ``distributed.tensor``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorplay_b200.distributed.tensor")
