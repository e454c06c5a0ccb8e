"""Expiration timers for worker code: PyTorch's module of the same role."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("torch.distributed.elastic.timer")
