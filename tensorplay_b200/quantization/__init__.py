"""Quantisation helpers: fp8 (e4m3 / e5m2) and int8 quantise / dequantise with per-tensor,
per-row or per-block scales (the reference ships fp8 as quantise/dequantise kernels only and
computes fp8 Linear as ``x @ dequant(w).T``, test/quantization/test_float8_modules.py:26-35)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def choose_scale_float8(x: torch.Tensor, dtype=torch.float8_e4m3fn, dim: Optional[int] = None) -> torch.Tensor:
    amax = x.abs().amax() if dim is None else x.abs().amax(dim=dim, keepdim=True)
    return (amax.float() / FP8_MAX[dtype]).clamp_(min=1e-12)


def quantize_affine_float8(x: torch.Tensor, scale: torch.Tensor, dtype=torch.float8_e4m3fn) -> torch.Tensor:
    from ..ops import fp8_quantize
    return fp8_quantize(x, scale, dtype)


def dequantize_affine_float8(q: torch.Tensor, scale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    from ..ops import fp8_dequantize
    return fp8_dequantize(q, scale, out_dtype)


def quantize_int8_rowwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    from ..ops import quantize_int8_rowwise as _q
    return _q(x)


def int8_mm_rescale(a_q, a_scale, w_q, w_scale, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``(a_q * a_scale) @ (w_q * w_scale).T`` with int32 accumulation (tcgen05 ``kind::i8`` on CUDA)."""
    from ..ops import int8_gemm
    return int8_gemm(a_q, w_q, a_scale, w_scale).to(out_dtype)


class Int8DynamicLinear(torch.nn.Module):
    """A8W8: activations quantised per row on the fly, weights per output channel, int8 tensor cores."""

    def __init__(self, linear: torch.nn.Linear):
        super().__init__()
        from ..ops import quantize_weight_int8
        q, s = quantize_weight_int8(linear.weight.data)
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s.float().reshape(-1))
        self.bias = linear.bias

    def forward(self, x):
        from ..ops import int8_gemm, quantize_int8_rowwise as _q
        x2 = x.reshape(-1, x.shape[-1])
        aq, asc = _q(x2.to(torch.bfloat16))
        y = int8_gemm(aq, self.qweight, asc, self.scale, self.bias)
        return y.view(*x.shape[:-1], -1).to(x.dtype)


class WeightOnlyLinear(torch.nn.Module):
    """W8A16 (per-channel or group-wise int8) or W4A16 (group-wise uint4) linear layer."""

    def __init__(self, linear: torch.nn.Linear, bits: int = 8, group_size: int = 0):
        super().__init__()
        from ..ops import quantize_weight_int4, quantize_weight_int8
        self.bits, self.group_size = bits, group_size
        if bits == 8:
            q, s = quantize_weight_int8(linear.weight.data, group_size)
            z = None
        elif bits == 4:
            self.group_size = group_size = group_size or 128
            q, s, z = quantize_weight_int4(linear.weight.data, group_size)
        else:
            raise ValueError("bits must be 8 or 4")
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s)
        self.register_buffer("zero", z)
        self.bias = linear.bias

    def forward(self, x):
        from ..ops import weight_only_linear
        return weight_only_linear(x, self.qweight, self.scale, self.zero, self.bias, self.bits, self.group_size)


def quantize_(module: torch.nn.Module, mode="int8_weight_only", group_size: int = 0,
              filter_fn=None) -> torch.nn.Module:
    """Swap every ``nn.Linear`` (accepted by ``filter_fn``) for its quantised counterpart in place.
    ``mode``: a recipe name (``int8_weight_only``, ``int4_weight_only``, ``int8_dynamic``, ``float8_weight_only``) or a
    configuration object / class of ``quantization.workflows`` (int8 mixed-precision training, the weight-only and fp8
    configurations, BitNet training)."""
    if not isinstance(mode, str):
        from .workflows import quantize_ as _by_config
        return _by_config(module, mode, filter_fn)
    make = {
        "int8_weight_only": lambda m: WeightOnlyLinear(m, 8, group_size),
        "int4_weight_only": lambda m: WeightOnlyLinear(m, 4, group_size or 128),
        "int8_dynamic": Int8DynamicLinear,
        "float8_weight_only": lambda m: Float8Linear(m),
    }[mode]
    for name, child in list(module.named_children()):
        if isinstance(child, torch.nn.Linear) and (filter_fn is None or filter_fn(child, name)):
            setattr(module, name, make(child))
        else:
            quantize_(child, mode, group_size, filter_fn)
    return module


class Float8Linear(torch.nn.Module):
    """Linear with fp8-stored weight, dequantised on the fly (weight-only fp8)."""

    def __init__(self, linear: torch.nn.Linear, dtype=torch.float8_e4m3fn):
        super().__init__()
        s = choose_scale_float8(linear.weight.data, dtype, dim=1)
        self.register_buffer("qweight", quantize_affine_float8(linear.weight.data, s, dtype))
        self.register_buffer("scale", s)
        self.bias = linear.bias

    def forward(self, x):
        from .. import ops
        w = dequantize_affine_float8(self.qweight, self.scale, x.dtype)
        return ops.linear(x, w, self.bias)


from .awq import AWQLinear, awq_quantize_, search_scales  # noqa: E402
from .pruning import (WeightSparsifier, compare_models, cubic_sparsity, global_magnitude_masks,  # noqa: E402
                      magnitude_mask, n_m_mask, sqnr)


from .bitnet import (BitNetLinear, BitNetPacked2bitLinearWeight, BitNetTrainingConfig, BitNetTrainingLinearWeight,  # noqa: E402,F401
                     bitnet_linear, bitnet_linear_packed, bitnet_training, pack_ternary, ternary_quantize, unpack_ternary)
from .workflows import *  # noqa: E402,F401,F403  (``quantize_`` above dispatches configuration objects to it)
