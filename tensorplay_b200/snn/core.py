"""The tau-parametrised LIF layer and its fused CUDA path: ``v <- v + (x - (v - v_reset)) / tau``,
hard reset, arctan surrogate; all time steps of a layer in one kernel launch (forward and BPTT)."""
from __future__ import annotations

import math

import torch
from torch import Tensor, nn

__all__ = ["spike", "LIFCell", "LIF", "rate_encode", "multi_step_lif"]


class _SpikeFn(torch.autograd.Function):
    """Heaviside forward, arctan surrogate derivative backward."""

    @staticmethod
    def forward(ctx, v, alpha):
        ctx.save_for_backward(v)
        ctx.alpha = alpha
        return (v >= 0).to(v.dtype)

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
        c = self.cell
        fused = multi_step_lif(x, c.tau, c.v_threshold, c.v_reset, c.alpha, c.detach_reset)
        if fused is not None:
            return fused
        v, out = None, []
        for t in range(x.shape[0]):
            s, v = self.cell(x[t], v)
            out.append(s)
        return torch.stack(out)


class _FusedLIFFn(torch.autograd.Function):
    """All time steps in one kernel launch; the forward keeps the pre-reset membrane (fp32) and the
    backward walks time in reverse over it (BPTT with the arctan surrogate)."""

    @staticmethod
    def forward(ctx, x, tau, v_th, v_reset, alpha, detach_reset):
        from .. import _native
        from ..ops._common import lib, ptr, stream_ptr
        steps, n = x.shape[0], x[0].numel()
        s = torch.empty_like(x)
        need = x.requires_grad
        h = torch.empty((steps, n), dtype=torch.float32, device=x.device) if need else None
        _native.check(lib().tpb_lif_fwd(ptr(x), ptr(s), ptr(h), None, steps, n, tau, v_th, v_reset,
                                        int(x.dtype == torch.bfloat16), stream_ptr()), "tpb_lif_fwd")
        ctx.save_for_backward(h)
        ctx.cfg = (tau, v_th, v_reset, alpha, detach_reset)
        return s

    @staticmethod
    def backward(ctx, gs):
        from .. import _native
        from ..ops._common import lib, ptr, stream_ptr
        (h,) = ctx.saved_tensors
        tau, v_th, v_reset, alpha, detach_reset = ctx.cfg
        gs = gs.contiguous()
        gx = torch.empty_like(gs)
        steps, n = h.shape
        _native.check(lib().tpb_lif_bwd(ptr(gs), ptr(h), ptr(gx), None, steps, n, tau, v_th, v_reset, alpha,
                                        int(detach_reset), int(gs.dtype == torch.bfloat16), stream_ptr()),
                      "tpb_lif_bwd")
        return gx, None, None, None, None, None


def multi_step_lif(x: Tensor, tau: float = 2.0, v_threshold: float = 1.0, v_reset: float = 0.0,
                   alpha: float = 2.0, detach_reset: bool = False):
    """Spikes ``[T, ...]`` of a LIF layer over the whole input sequence ``x [T, ...]`` by the fused
    CUDA kernel, or ``None`` when the input does not qualify (CPU tensor, other dtype, neuron count
    not a multiple of 4): the caller then loops over :class:`LIFCell`."""
    from ..ops._common import use_native
    if not (x.is_cuda and use_native(x) and x.dtype in (torch.float32, torch.bfloat16) and x.dim() >= 2
            and x[0].numel() % 4 == 0):
        return None
    return _FusedLIFFn.apply(x.contiguous(), float(tau), float(v_threshold), float(v_reset), float(alpha),
                             bool(detach_reset))


def rate_encode(x: Tensor, steps: int, generator=None) -> Tensor:
    """Bernoulli spike trains ``[steps, ...]`` with firing probability ``x`` in [0, 1]."""
    return (torch.rand((steps,) + tuple(x.shape), device=x.device, generator=generator) < x).to(x.dtype)
