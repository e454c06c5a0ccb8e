"""``ao``: PyTorch's architecture-optimisation package (quantisation workflows, pruning, sparsity) with this framework's
additions under ``ao.quantization`` (BitNet b1.58 layers, the fp8 / int8 / int4 helpers of ``tensorplay_b200.quantization``).
Sub-module paths without a file here resolve to ``torch.ao``'s modules as the same objects."""
from . import quantization  # noqa: F401


def __getattr__(name):
    import importlib
    import torch.ao as _ao
    try:
        return getattr(_ao, name)
    except AttributeError:
        try:
            return importlib.import_module(f"torch.ao.{name}")
        except ImportError:
            raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
