"""Layers for sequences of spikes (the reference's ``tensorplay/snn/layer.py``): fold time into the
batch for stateless layers."""
from __future__ import annotations

from torch import Tensor, nn


class SeqToANNContainer(nn.Sequential):
    """Applies stateless layers to ``[T, B, ...]`` by folding time into the batch dimension."""

    def forward(self, x: Tensor) -> Tensor:
        t, b = x.shape[0], x.shape[1]
        y = super().forward(x.flatten(0, 1))
        return y.view(t, b, *y.shape[1:])


class SpikingConv2d(SeqToANNContainer):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, bias: bool = False):
        super().__init__(nn.Conv2d(in_channels, out_channels, kernel_size, stride, padding, bias=bias))


class SpikingBatchNorm1d(SeqToANNContainer):
    """Batch statistics over time and batch together (time folded into the batch)."""

    def __init__(self, num_features: int, **kw):
        super().__init__(nn.BatchNorm1d(num_features, **kw))


class SpikingBatchNorm2d(SeqToANNContainer):
    def __init__(self, num_features: int, **kw):
        super().__init__(nn.BatchNorm2d(num_features, **kw))
