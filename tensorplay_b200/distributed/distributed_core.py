"""``distributed.distributed_core``: the process-group and collective API, which this package exposes at its top level."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("tensorplay_b200.distributed")
