"""Spiking neural network primitives (the ``tensorplay.snn`` pack): neuron models, surrogate
gradients, spike encoders, sequence layers and monitoring.

    >>> from tensorplay_b200 import snn
    >>> lif = snn.LIFNode(threshold=1.0, decay=0.5)          # single-step, state kept in lif.v
    >>> seq = snn.LIFNode(step_mode="m", surrogate=snn.ATanSurrogate())
    >>> out = seq(torch.rand(8, 4, 16))                      # [T, B, N] spike train
    >>> fast = snn.LIF(tau=2.0)                              # all steps in one CUDA launch on a B200
"""
from . import encoding, functional, layer, monitor, surrogate
from .core import LIF, LIFCell, multi_step_lif
from .core import spike as atan_spike
from .encoding import (GaussianTuningCurveEncoder, LatencyEncoder, PeriodicEncoder, WeightedPhaseEncoder,
                       poisson_encode, rate_encode, temporal_encode)
from .functional import heaviside, lif_seq, lif_step, spike_rate, spike_rate_loss, surrogate_grad
from .layer import SeqToANNContainer, SpikingBatchNorm1d, SpikingBatchNorm2d, SpikingConv2d
from .monitor import SpikeMonitor
from .neuron import ALIFNode, IFNode, LIFNode, ParametricLIFNode, SpikeLinear
from .surrogate import *  # noqa: F401,F403
from .surrogate import SURROGATES, SurrogateBase


def spike(v, alpha_or_surrogate=2.0):
    """Heaviside step of ``v`` with a surrogate derivative: a number selects the arctan surrogate of
    that ``alpha`` (the fused kernel's), a surrogate object is used as given."""
    if isinstance(alpha_or_surrogate, SurrogateBase):
        return alpha_or_surrogate(v)
    return atan_spike(v, float(alpha_or_surrogate))
