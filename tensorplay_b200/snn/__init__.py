"""Spiking neural network layers: leaky integrate-and-fire neurons trained with surrogate
gradients (the reference's ``tensorplay.snn`` pack: tensorplay/snn/__init__.py)."""
from __future__ import annotations

import math

import torch
from torch import Tensor, nn

__all__ = ["spike", "LIFCell", "LIF", "rate_encode"]


class _SpikeFn(torch.autograd.Function):
    """Heaviside forward, arctan surrogate derivative backward."""

    @staticmethod
    def forward(ctx, v, alpha):
        ctx.save_for_backward(v)
        ctx.alpha = alpha
        return (v > 0).to(v.dtype)

    @staticmethod
    def backward(ctx, g):
        (v,) = ctx.saved_tensors
        a = ctx.alpha
        return g * (a / 2) / (1 + (math.pi / 2 * a * v) ** 2), None


def spike(v: Tensor, alpha: float = 2.0) -> Tensor:
    return _SpikeFn.apply(v, alpha)


class LIFCell(nn.Module):
    """One step of a leaky integrate-and-fire neuron: ``v <- v + (x - (v - v_reset)) / tau``,
    spike where ``v >= v_threshold``, hard reset to ``v_reset``."""

    def __init__(self, tau: float = 2.0, v_threshold: float = 1.0, v_reset: float = 0.0, alpha: float = 2.0,
                 detach_reset: bool = False) -> None:
        super().__init__()
        self.tau, self.v_threshold, self.v_reset, self.alpha = tau, v_threshold, v_reset, alpha
        self.detach_reset = detach_reset

    def forward(self, x: Tensor, v: Tensor = None):
        if v is None:
            v = torch.full_like(x, self.v_reset)
        v = v + (x - (v - self.v_reset)) / self.tau
        s = spike(v - self.v_threshold, self.alpha)
        r = s.detach() if self.detach_reset else s
        v = v * (1 - r) + self.v_reset * r
        return s, v


class LIF(nn.Module):
    """Runs :class:`LIFCell` over the leading time dimension ``[T, ...]``."""

    def __init__(self, **kw) -> None:
        super().__init__()
        self.cell = LIFCell(**kw)

    def forward(self, x: Tensor) -> Tensor:
        v, out = None, []
        for t in range(x.shape[0]):
            s, v = self.cell(x[t], v)
            out.append(s)
        return torch.stack(out)


def rate_encode(x: Tensor, steps: int, generator=None) -> Tensor:
    """Bernoulli spike trains ``[steps, ...]`` with firing probability ``x`` in [0, 1]."""
    return (torch.rand((steps,) + tuple(x.shape), device=x.device, generator=generator) < x).to(x.dtype)
