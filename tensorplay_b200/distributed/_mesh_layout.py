"""Mesh layout algebra: PyTorch's module of the same role."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("torch.distributed._mesh_layout")
