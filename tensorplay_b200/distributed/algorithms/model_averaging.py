"""Periodic and hierarchical model averaging: PyTorch's package of the same role."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("torch.distributed.algorithms.model_averaging")
