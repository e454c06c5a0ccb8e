"""``cuda``: device management, streams/events, memory stats and CUDA graphs (torch.cuda), plus
the graph-capture helper used instead of a tracing compiler."""
from torch.cuda import *  # noqa: F401,F403
from torch.cuda import (CUDAGraph, Event, Stream, current_device, current_stream, device_count,  # noqa: F401
                        graph, is_available, make_graphed_callables, memory_allocated, nvtx,
                        set_device, synchronize)
import torch.cuda as _tc

from . import graphs  # noqa: F401


def __getattr__(name):
    return getattr(_tc, name)


# ---- names of the reference's ``cuda`` package without a same-named counterpart in torch.cuda
def is_gds_available() -> bool:
    """GPUDirect Storage entry points (``torch.cuda.gds``) are usable only with a cuFile-enabled build."""
    try:
        from torch.cuda import gds
        return hasattr(gds, "GdsFile") and is_available()
    except Exception:
        return False


def current_solver_handle():
    """cuSOLVER handle of the current stream (the linear-algebra library handle of this device)."""
    import torch
    return torch.cuda.current_blas_handle() if not hasattr(_tc, "current_solver_handle") else _tc.current_solver_handle()


class caching_allocator_disabled:
    """Context manager: allocations inside bypass the caching allocator's reuse by emptying the
    cache on entry and exit (diagnostic mode for memory tools; the allocator itself stays on)."""

    def __enter__(self):
        if is_available():
            _tc.empty_cache()
        return self

    def __exit__(self, *exc):
        if is_available():
            _tc.empty_cache()
        return False


def export_dot(graph_obj, path: str) -> str:
    """Write a captured CUDA graph as Graphviz DOT (``CUDAGraph.debug_dump``; needs ``enable_debug_mode``
    before capture)."""
    graph_obj.debug_dump(path)
    return path


class graph_annotations:
    """NVTX range around a graph capture so that the captured region is named in timelines."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if is_available():
            _tc.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if is_available():
            _tc.nvtx.range_pop()
        return False


def __getattr__(name):  # noqa: F811
    if name == "GdsFile":
        from torch.cuda import gds
        return gds.GdsFile
    return getattr(_tc, name)

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("graph_annotations",))
