"""Spike statistics of a network's neuron layers (the reference's ``tensorplay/snn/monitor.py``)."""
from __future__ import annotations

from typing import Dict, List

import torch
from torch import nn


class SpikeMonitor:
    """Forward hooks on the neuron modules of ``net`` that accumulate spike counts and element counts.

    ``rates()`` gives the mean firing rate per monitored layer; ``reset()`` clears the counters;
    ``remove()`` detaches the hooks (also on leaving a ``with`` block).
    """

    def __init__(self, net: nn.Module, types=None):
        from .core import LIF, LIFCell
        from .neuron import LIFNode
        types = tuple(types) if types is not None else (LIFNode, LIF, LIFCell)
        self.counts: Dict[str, float] = {}
        self.numel: Dict[str, int] = {}
        self.handles: List = []
        for name, m in net.named_modules():
            if isinstance(m, types):
                self.handles.append(m.register_forward_hook(self._hook(name)))

    def _hook(self, name: str):
        def fn(mod, inp, out):
            s = out[0] if isinstance(out, tuple) else out
            self.counts[name] = self.counts.get(name, 0.0) + float(s.detach().sum())
            self.numel[name] = self.numel.get(name, 0) + s.numel()
        return fn

    def rates(self) -> Dict[str, float]:
        return {k: self.counts[k] / max(1, self.numel[k]) for k in self.counts}

    def reset(self) -> None:
        self.counts.clear()
        self.numel.clear()

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()
