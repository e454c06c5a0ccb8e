"""Quantised collectives by decoration (tensorplay/distributed/algorithms/_quantization): PyTorch's ``auto_quantize`` and
``DQuantType``; the gradient-compression hooks of this framework are ``algorithms.quantization_pertensor_hook`` /
``quantization_perchannel_hook``."""
from torch.distributed.algorithms._quantization.quantization import DQuantType, auto_quantize

__all__ = ["DQuantType", "auto_quantize"]
