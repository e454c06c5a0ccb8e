"""Neuron modules (the reference's ``tensorplay/snn/neuron.py``): LIF, IF, parametric LIF, adaptive
LIF and the bias-free ``SpikeLinear``; single-step (``"s"``) and multi-step (``"m"``) modes."""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import Tensor, nn

from .functional import lif_seq, lif_step, spike
from .surrogate import StraightThroughSurrogate, SurrogateBase


class LIFNode(nn.Module):
    """Leaky integrate-and-fire neuron with state ``v`` kept between calls (``reset()`` clears it)."""

    def __init__(self, threshold=1.0, decay=0.5, v_reset: Optional[float] = 0.0,
                 surrogate: Optional[SurrogateBase] = None, detach_reset: bool = True, step_mode: str = "s",
                 learnable_threshold: bool = False, return_v_seq: bool = False) -> None:
        super().__init__()
        self.threshold = nn.Parameter(torch.tensor(float(threshold))) if learnable_threshold else threshold
        self.decay, self.v_reset = decay, v_reset
        self.surrogate = surrogate if surrogate is not None else StraightThroughSurrogate()
        self.detach_reset, self.step_mode, self.return_v_seq = detach_reset, step_mode, return_v_seq
        self.v: Optional[Tensor] = None

    def reset(self) -> None:
        self.v = None

    def detach(self) -> None:
        if self.v is not None:
            self.v = self.v.detach()

    def _decay(self):
        return self.decay

    def _state(self, ref: Tensor) -> Optional[Tensor]:
        if self.v is None or self.v.shape != ref.shape:
            return None
        return self.v

    def forward(self, x: Tensor):
        if self.step_mode == "s":
            v = self._state(x)
            s, self.v = lif_step(x, torch.zeros_like(x) if v is None else v, self._decay(), self.threshold,
                                 self.v_reset, self.surrogate, self.detach_reset)
            return s
        if self.step_mode != "m":
            raise ValueError(f"step_mode must be 's' or 'm', got {self.step_mode!r}")
        if x.dim() < 2:
            raise ValueError("multi-step input must have shape [T, B, ...]")
        out = lif_seq(x, self._state(x[0]), self._decay(), self.threshold, self.v_reset, self.surrogate,
                      self.detach_reset, self.return_v_seq)
        self.v = out[-1]
        return (out[0], out[1]) if self.return_v_seq else out[0]

    def extra_repr(self) -> str:
        return f"threshold={self.threshold}, decay={self.decay}, v_reset={self.v_reset}, step_mode={self.step_mode}"


class IFNode(LIFNode):
    """Integrate-and-fire: no leak (``decay = 1``)."""

    def __init__(self, threshold=1.0, v_reset: Optional[float] = 0.0, **kw) -> None:
        super().__init__(threshold=threshold, decay=1.0, v_reset=v_reset, **kw)


class ParametricLIFNode(LIFNode):
    """LIF whose leak is learned: ``decay = sigmoid(w)``, initialised to ``init_decay``."""

    def __init__(self, threshold=1.0, init_decay: float = 0.5, **kw) -> None:
        super().__init__(threshold=threshold, decay=init_decay, **kw)
        self.w = nn.Parameter(torch.tensor(math.log(init_decay / (1 - init_decay))))

    def _decay(self):
        return torch.sigmoid(self.w)


class ALIFNode(LIFNode):
    """Adaptive LIF: every spike raises the threshold by ``beta`` through a trace ``a`` that decays
    with ``rho``: ``a <- rho a + s``, effective threshold ``threshold + beta a``."""

    def __init__(self, threshold=1.0, decay=0.5, rho: float = 0.9, beta: float = 0.2, **kw) -> None:
        super().__init__(threshold=threshold, decay=decay, **kw)
        self.rho, self.beta = rho, beta
        self.a: Optional[Tensor] = None

    def reset(self) -> None:
        super().reset()
        self.a = None

    def _one(self, x: Tensor) -> Tensor:
        if self.v is None or self.v.shape != x.shape:
            self.v = torch.zeros_like(x)
        if self.a is None or self.a.shape != x.shape:
            self.a = torch.zeros_like(x)
        s, self.v = lif_step(x, self.v, self.decay, self.threshold + self.beta * self.a, self.v_reset,
                             self.surrogate, self.detach_reset)
        self.a = self.rho * self.a + s.detach()
        return s

    def forward(self, x: Tensor):
        if self.step_mode == "s":
            return self._one(x)
        return torch.stack([self._one(x[t]) for t in range(x.shape[0])])


class SpikeLinear(nn.Module):
    """Linear synapse layer for spike trains (no bias by default: silent inputs give no current)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False) -> None:
        super().__init__()
        self.linear = nn.Linear(in_features, out_features, bias=bias)

    def forward(self, x: Tensor) -> Tensor:
        return self.linear(x)
