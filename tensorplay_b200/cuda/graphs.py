"""CUDA-graph capture of a module's forward for static shapes.

The kernels of this package are launched on ``torch.cuda.current_stream()`` and encode their
TMA descriptors on the host at launch time, so they are capturable like any other launch.
(API after tensorplay/cuda/graphs.py:82-563: ``CUDAGraph``, ``graph``, ``make_graphed_callables``.)
"""
from __future__ import annotations

import torch
from torch.cuda import CUDAGraph, graph, make_graphed_callables  # noqa: F401


class _Graphed:
    def __init__(self, fn):
        self.fn = fn
        self.cache = {}

    def __call__(self, *args):
        if torch.is_grad_enabled() and any(isinstance(a, torch.Tensor) and a.requires_grad for a in args):
            return self.fn(*args)
        key = tuple((tuple(a.shape), a.dtype) if isinstance(a, torch.Tensor) else a for a in args)
        ent = self.cache.get(key)
        if ent is None:
            static_in = [a.clone() if isinstance(a, torch.Tensor) else a for a in args]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s), torch.no_grad():
                for _ in range(2):
                    self.fn(*static_in)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g), torch.no_grad():
                out = self.fn(*static_in)
            ent = (g, static_in, out)
            self.cache[key] = ent
        g, static_in, out = ent
        for dst, src in zip(static_in, args):
            if isinstance(dst, torch.Tensor):
                dst.copy_(src)
        g.replay()
        return out

    def __getattr__(self, name):
        return getattr(self.fn, name)


def make_graphed_callable(fn):
    """Wrap ``fn`` so that inference calls with a repeated input signature replay a CUDA graph."""
    return _Graphed(fn)
