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
