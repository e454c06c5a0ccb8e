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
    return (x.float() / scale).clamp_(-FP8_MAX[dtype], FP8_MAX[dtype]).to(dtype)


def dequantize_affine_float8(q: torch.Tensor, scale: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    return (q.float() * scale).to(out_dtype)


def quantize_int8_rowwise(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    scale = x.float().abs().amax(dim=-1, keepdim=True).clamp_(min=1e-8) / 127.0
    return torch.clamp(torch.round(x.float() / scale), -127, 127).to(torch.int8), scale


def int8_mm_rescale(a_q, a_scale, w_q, w_scale, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``(a_q * a_scale) @ (w_q * w_scale).T`` with int32 accumulation."""
    acc = torch._int_mm(a_q, w_q.t().contiguous()) if a_q.is_cuda and a_q.shape[0] > 16 else a_q.int() @ w_q.int().t()
    return (acc.float() * a_scale * w_scale.reshape(1, -1)).to(out_dtype)


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
