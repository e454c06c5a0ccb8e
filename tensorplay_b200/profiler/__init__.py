"""``profiler``: torch.profiler plus NVTX range helpers and a launch counter for our kernels."""
from torch.profiler import *  # noqa: F401,F403
from torch.profiler import ProfilerActivity, profile, record_function, schedule, tensorboard_trace_handler  # noqa: F401

from .. import _native


def kernel_launches() -> int:
    """Number of launches of this package's kernels so far in the process."""
    return _native.launch_count


class nvtx_range:
    """Context manager pushing an NVTX range (visible in Nsight tools)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


def __getattr__(name):
    """Event containers, ``emit_nvtx`` / ``emit_itt`` and the rest of the profiler surface resolve to PyTorch's."""
    import importlib
    for mod in ['torch.profiler', 'torch.autograd.profiler', 'torch.autograd.profiler_util', 'torch.cuda.nvtx']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
