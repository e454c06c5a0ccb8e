"""Spike encoders (the reference's ``tensorplay/snn/encoding.py``): rate / Poisson, latency,
weighted phase, periodic and Gaussian tuning curves."""
from __future__ import annotations

import math

import torch
from torch import Tensor


def rate_encode(x: Tensor, steps: int, generator=None) -> Tensor:
    """Bernoulli spike trains ``[steps, ...]`` with firing probability ``x`` in [0, 1]."""
    return (torch.rand((steps,) + tuple(x.shape), device=x.device, generator=generator) < x).to(x.dtype)


poisson_encode = rate_encode


def temporal_encode(x: Tensor, steps: int) -> Tensor:
    """Time-to-first-spike: one spike per element, earlier for larger ``x`` in [0, 1]."""
    t = ((1 - x.clamp(0, 1)) * (steps - 1)).round().long()
    out = torch.zeros((steps,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    return out.scatter_(0, t.unsqueeze(0), 1.0)


class LatencyEncoder:
    """Spike at step ``round((T - 1) (1 - x))`` (linear) or ``round((T - 1) - ln(alpha x + 1))`` (log)."""

    def __init__(self, steps: int, kind: str = "linear", alpha: float = None):
        self.steps, self.kind = steps, kind
        self.alpha = alpha if alpha is not None else math.exp(steps - 1) - 1

    def __call__(self, x: Tensor) -> Tensor:
        if self.kind == "linear":
            return temporal_encode(x, self.steps)
        t = ((self.steps - 1) - torch.log(self.alpha * x.clamp(0, 1) + 1)).round().clamp(0, self.steps - 1).long()
        out = torch.zeros((self.steps,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        return out.scatter_(0, t.unsqueeze(0), 1.0)


class WeightedPhaseEncoder:
    """Binary expansion of ``x`` in [0, 1): step ``k`` carries the bit of weight ``2^-(k+1)``."""

    def __init__(self, phases: int = 8):
        self.phases = phases

    def __call__(self, x: Tensor) -> Tensor:
        rem, out = x.clamp(0, 1 - 2.0 ** -self.phases).clone(), []
        for k in range(self.phases):
            w = 2.0 ** -(k + 1)
            bit = (rem >= w).to(x.dtype)
            out.append(bit)
            rem = rem - bit * w
        return torch.stack(out)

    def decode(self, spikes: Tensor) -> Tensor:
        w = torch.tensor([2.0 ** -(k + 1) for k in range(self.phases)], dtype=spikes.dtype, device=spikes.device)
        return (spikes * w.view(-1, *([1] * (spikes.dim() - 1)))).sum(0)


class PeriodicEncoder:
    """Replays a fixed spike pattern ``[P, ...]`` cyclically."""

    def __init__(self, pattern: Tensor):
        self.pattern = pattern

    def __call__(self, steps: int) -> Tensor:
        idx = torch.arange(steps, device=self.pattern.device) % self.pattern.shape[0]
        return self.pattern[idx]


class GaussianTuningCurveEncoder:
    """Population code: ``m`` neurons with Gaussian receptive fields over ``[x_min, x_max]``; the
    response strength sets the spike latency within ``steps``."""

    def __init__(self, x_min: float, x_max: float, m: int, steps: int, beta: float = 1.5):
        self.steps, self.m = steps, m
        self.mu = x_min + (2 * torch.arange(1, m + 1) - 3) / 2 * (x_max - x_min) / (m - 2)
        self.sigma = (x_max - x_min) / (beta * (m - 2))

    def __call__(self, x: Tensor) -> Tensor:
        mu = self.mu.to(x.device, x.dtype)
        resp = torch.exp(-((x.unsqueeze(-1) - mu) ** 2) / (2 * self.sigma ** 2))    # [..., m] in (0, 1]
        return temporal_encode(resp, self.steps)
