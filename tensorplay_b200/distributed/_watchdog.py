"""The watchdog under the reference's private module path (tensorplay/distributed/_watchdog.py)."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorplay_b200.distributed.watchdog")
