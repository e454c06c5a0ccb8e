"""Process start / tee / error files of the elastic agent: PyTorch's module of the same role."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("torch.distributed.elastic.multiprocessing")
