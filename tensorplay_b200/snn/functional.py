"""Functional spiking primitives (the reference's ``tensorplay/snn/functional.py``): one LIF step,
a whole sequence, spike rates and the rate loss.

    h = decay * v + x;  s = (h >= threshold);  v' = h - threshold * s   (soft reset, v_reset None)
                                               v' = h (1 - s) + v_reset s   (hard reset)
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .surrogate import StraightThroughSurrogate, SurrogateBase


def heaviside(x: Tensor) -> Tensor:
    """Spike step: 1 where ``x >= 0``, 0 elsewhere."""
    return (x >= 0).to(x.dtype)


def spike(u: Tensor, surrogate: Optional[SurrogateBase] = None) -> Tensor:
    return (surrogate or StraightThroughSurrogate())(u)


def surrogate_grad(u: Tensor, surrogate: Optional[SurrogateBase] = None) -> Tensor:
    return (surrogate or StraightThroughSurrogate()).grad(u)


def lif_step(x: Tensor, v: Tensor, decay=0.5, threshold=1.0, v_reset: Optional[float] = 0.0,
             surrogate: Optional[SurrogateBase] = None, detach_reset: bool = True):
    """One step; returns ``(spike, v_new)``. ``decay`` / ``threshold`` may be tensors (learnable)."""
    h = decay * v + x
    s = spike(h - threshold, surrogate)
    r = s.detach() if detach_reset else s
    if v_reset is None:
        v_new = h - threshold * r
    else:
        v_new = h * (1 - r) + v_reset * r
    return s, v_new


def lif_seq(x: Tensor, v_init: Optional[Tensor] = None, decay=0.5, threshold=1.0, v_reset: Optional[float] = 0.0,
            surrogate: Optional[SurrogateBase] = None, detach_reset: bool = True, return_v_seq: bool = False):
    """All steps of ``x [T, ...]``: ``(spikes, v_final)`` or ``(spikes, v_seq, v_final)``, through
    autograd. (The one-launch CUDA version of the fixed configuration - hard reset, arctan surrogate,
    zero initial membrane - is :func:`tensorplay_b200.snn.multi_step_lif` / :class:`tensorplay_b200.snn.LIF`.)"""
    v = torch.zeros_like(x[0]) if v_init is None else v_init
    spikes, vs = [], []
    for t in range(x.shape[0]):
        s, v = lif_step(x[t], v, decay, threshold, v_reset, surrogate, detach_reset)
        spikes.append(s)
        if return_v_seq:
            vs.append(v)
    if return_v_seq:
        return torch.stack(spikes), torch.stack(vs), v
    return torch.stack(spikes), v


def spike_rate(spikes: Tensor, dim: int = 0) -> Tensor:
    """Mean firing rate over the time axis."""
    return spikes.float().mean(dim)


def spike_rate_loss(spikes: Tensor, target_rate, dim: int = 0) -> Tensor:
    """Mean squared distance between the firing rates and a target rate (scalar or tensor)."""
    return ((spike_rate(spikes, dim) - target_rate) ** 2).mean()
