"""Surrogate gradients of the spike step (the reference's ``tensorplay/snn/surrogate.py``: the
forward is always the Heaviside step, each class supplies the derivative used in backward)."""
from __future__ import annotations

import math

import torch
from torch import Tensor


class SurrogateBase:
    """Callable ``s = surrogate(u)`` with ``u = h - threshold``: Heaviside forward, ``grad(u)`` backward."""

    def grad(self, u: Tensor) -> Tensor:
        raise NotImplementedError

    def __call__(self, u: Tensor) -> Tensor:
        return _Spike.apply(u, self)

    def __repr__(self) -> str:
        args = ", ".join(f"{k}={v}" for k, v in vars(self).items())
        return f"{type(self).__name__}({args})"


class _Spike(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, surrogate):
        ctx.save_for_backward(u)
        ctx.surrogate = surrogate
        return (u >= 0).to(u.dtype)

    @staticmethod
    def backward(ctx, g):
        (u,) = ctx.saved_tensors
        return g * ctx.surrogate.grad(u), None


class StraightThroughSurrogate(SurrogateBase):
    """Gradient 1 inside a window of half-width ``w`` around the threshold, 0 outside."""

    def __init__(self, w: float = 1.0):
        self.w = w

    def grad(self, u):
        return (u.abs() <= self.w).to(u.dtype)


class SigmoidSurrogate(SurrogateBase):
    def __init__(self, alpha: float = 4.0):
        self.alpha = alpha

    def grad(self, u):
        s = torch.sigmoid(self.alpha * u)
        return self.alpha * s * (1 - s)


class FastSigmoidSurrogate(SurrogateBase):
    """``1 / (1 + alpha |u|)^2`` (SuperSpike's shape with unit height)."""

    def __init__(self, alpha: float = 2.0):
        self.alpha = alpha

    def grad(self, u):
        return 1.0 / (1.0 + self.alpha * u.abs()) ** 2


class SuperSpikeSurrogate(FastSigmoidSurrogate):
    def __init__(self, beta: float = 10.0):
        super().__init__(beta)


class ATanSurrogate(SurrogateBase):
    """``(alpha / 2) / (1 + (pi / 2 alpha u)^2)``: the derivative the fused LIF kernel uses."""

    def __init__(self, alpha: float = 2.0):
        self.alpha = alpha

    def grad(self, u):
        return (self.alpha / 2) / (1 + (math.pi / 2 * self.alpha * u) ** 2)


class ErfSurrogate(SurrogateBase):
    """Gaussian bump, the derivative of ``erfc``-shaped smoothing."""

    def __init__(self, alpha: float = 2.0):
        self.alpha = alpha

    def grad(self, u):
        return self.alpha / math.sqrt(math.pi) * torch.exp(-(self.alpha * u) ** 2)


class PiecewiseLinearSurrogate(SurrogateBase):
    """Triangle of height ``alpha`` and half-width ``1 / alpha``."""

    def __init__(self, alpha: float = 1.0):
        self.alpha = alpha

    def grad(self, u):
        return (self.alpha - self.alpha ** 2 * u.abs()).clamp(min=0)


class PiecewiseQuadraticSurrogate(SurrogateBase):
    """Derivative of the piecewise-quadratic smoothing: a triangle ``alpha (1 - alpha |u|)`` as well,
    normalised to unit area (kept as its own class for parity of configurations)."""

    def __init__(self, alpha: float = 1.0):
        self.alpha = alpha

    def grad(self, u):
        return (self.alpha * (1 - self.alpha * u.abs())).clamp(min=0)


class PiecewiseExpSurrogate(SurrogateBase):
    def __init__(self, alpha: float = 2.0):
        self.alpha = alpha

    def grad(self, u):
        return self.alpha / 2 * torch.exp(-self.alpha * u.abs())


class NonzeroSignLogAbsSurrogate(SurrogateBase):
    """``1 / (1 + alpha |u|)``: the derivative of ``sign(u) log(alpha |u| + 1) / alpha``."""

    def __init__(self, alpha: float = 1.0):
        self.alpha = alpha

    def grad(self, u):
        return 1.0 / (1.0 + self.alpha * u.abs())


class PiecewiseLeakyRELUSurrogate(SurrogateBase):
    """Slope ``1 / w`` inside ``|u| < w``, leak ``c`` outside."""

    def __init__(self, w: float = 1.0, c: float = 0.01):
        self.w, self.c = w, c

    def grad(self, u):
        inside = (u.abs() < self.w).to(u.dtype)
        return inside / self.w + (1 - inside) * self.c


class LeakyKRELUSurrogate(SurrogateBase):
    """Slope ``k`` for ``u >= 0`` and ``leak`` below."""

    def __init__(self, leak: float = 0.0, k: float = 1.0):
        self.leak, self.k = leak, k

    def grad(self, u):
        pos = (u >= 0).to(u.dtype)
        return pos * self.k + (1 - pos) * self.leak


class S2NNSurrogate(SurrogateBase):
    """Sigmoid derivative below the threshold, ``beta / (u + 1)`` above (single-step SNN training)."""

    def __init__(self, alpha: float = 4.0, beta: float = 1.0):
        self.alpha, self.beta = alpha, beta

    def grad(self, u):
        s = torch.sigmoid(self.alpha * u)
        below = self.alpha * s * (1 - s)
        above = self.beta / (u.clamp(min=0) + 1)
        return torch.where(u < 0, below, above)


class QPseudoSpikeSurrogate(SurrogateBase):
    """``(1 + 2 |u| / (alpha - 1))^(-alpha)`` with ``alpha > 1`` (heavy-tailed)."""

    def __init__(self, alpha: float = 2.0):
        self.alpha = alpha

    def grad(self, u):
        return (1 + 2 * u.abs() / (self.alpha - 1)) ** (-self.alpha)


class FourierSeriesSurrogate(SurrogateBase):
    """Derivative of the ``n``-term Fourier series of a square wave of period ``T_period``."""

    def __init__(self, n: int = 2, T_period: float = 8.0):
        self.n, self.T_period = n, T_period

    def grad(self, u):
        w0 = 2 * math.pi / self.T_period
        out = torch.zeros_like(u)
        for i in range(1, self.n + 1):
            out = out + torch.cos((2 * i - 1) * w0 * u)
        return out * (4 / self.T_period)


SURROGATES = {c.__name__: c for c in (
    StraightThroughSurrogate, SigmoidSurrogate, FastSigmoidSurrogate, PiecewiseLinearSurrogate, ATanSurrogate,
    ErfSurrogate, PiecewiseQuadraticSurrogate, PiecewiseExpSurrogate, SuperSpikeSurrogate,
    NonzeroSignLogAbsSurrogate, PiecewiseLeakyRELUSurrogate, LeakyKRELUSurrogate, S2NNSurrogate,
    QPseudoSpikeSurrogate, FourierSeriesSurrogate)}

SquarewaveFourierSeriesSurrogate = FourierSeriesSurrogate
SURROGATES["SquarewaveFourierSeriesSurrogate"] = FourierSeriesSurrogate
