"""``ao.quantization``: PyTorch's quantisation workflows, the functional spellings that the reference lists here
(``quantize_per_tensor``, ``dequantize``, ``q_scale`` ...: PyTorch keeps them at its top level or as tensor methods), and
this framework's BitNet b1.58 layers and weight-only / fp8 helpers (tensorplay/ao/quantization/__init__.py)."""
import torch as _torch
import torch.ao.quantization  # noqa: F401

# (no star import: PyTorch's ``__all__`` here names things the module does not define)
globals().update({_n: getattr(_torch.ao.quantization, _n) for _n in dir(_torch.ao.quantization) if not _n.startswith("_")})

from ..quantization import bitnet as _bitnet
from ..quantization.bitnet import *  # noqa: F401,F403
from ..quantization.workflows import *  # noqa: F401,F403
from ..quantization import quantize_  # noqa: F401  (recipe names and configuration objects)


def dequantize(t):
    return t.dequantize()


def int_repr(t):
    return t.int_repr()


def is_quantized(t) -> bool:
    return bool(t.is_quantized)


def q_scale(t) -> float:
    return t.q_scale()


def q_zero_point(t) -> int:
    return t.q_zero_point()


def q_per_channel_scales(t):
    return t.q_per_channel_scales()


def q_per_channel_zero_points(t):
    return t.q_per_channel_zero_points()


def q_per_channel_axis(t) -> int:
    return t.q_per_channel_axis()


def qscheme(t):
    return t.qscheme()


def fake_quantize_per_tensor(x, scale, zero_point, quant_min, quant_max):
    return _torch.fake_quantize_per_tensor_affine(x, scale, zero_point, quant_min, quant_max)


def fake_quantize_per_channel(x, scale, zero_point, axis, quant_min, quant_max):
    return _torch.fake_quantize_per_channel_affine(x, scale, zero_point, axis, quant_min, quant_max)


def quantized_linear(x, weight, bias=None, scale: float = 1.0, zero_point: int = 0):
    """Quantised ``x`` and weight -> quantised output (PyTorch's quantised linear kernel)."""
    return _torch.ao.nn.quantized.functional.linear(x, weight, bias, scale, zero_point)


def quantized_linear_dynamic(x, weight, bias=None):
    """Float ``x``, int8 weight-only: per-row activation quantisation, integer product, float output
    (this framework's int8 path)."""
    from .. import ops
    a_q, a_s = ops.quantize_int8_rowwise(x)
    w_q, w_s = ops.quantize_weight_int8(weight)
    return ops.int8_gemm(a_q.reshape(-1, a_q.shape[-1]), w_q, a_s, w_s, bias).reshape(*x.shape[:-1], -1)


def __getattr__(name):
    import importlib
    for ns in (_torch.ao.quantization, _torch, _bitnet):
        if hasattr(ns, name):
            return getattr(ns, name)
    if name == "PerChannelFakeQuantize":
        return _torch.ao.quantization.FakeQuantize
    if name == "default_per_channel_qat_qconfig":
        return _torch.ao.quantization.qconfig.default_per_channel_symmetric_qnnpack_qat_qconfig
    pkg = importlib.import_module("tensorplay_b200.quantization")
    if hasattr(pkg, name):
        return getattr(pkg, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
