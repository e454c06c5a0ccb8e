"""Quantised linear algebra: int8 tensor-core GEMM (A8W8 rowwise), weight-only GEMV / GEMM
(W8A16, W4A16 group-wise) and fp8 / int8 quantise-dequantise.

CUDA tensors run the kernels of ``csrc/kernels/quant_ops.cu``; CPU tensors run the plain
PyTorch expressions below, which are also the oracle of the GPU tests. Capability reference:
p10/src/backend/cuda/QuantGemmKernels.cu:92-1611, IntMM.cu:62, AffineQuantKernels.cu:1302.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native
from ._common import lib, ptr, status_word, stream_ptr, use_native

_FP8 = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
_FP8_MAX = {torch.float8_e4m3fn: 448.0, torch.float8_e5m2: 57344.0}


def quantize_int8_rowwise(x: Tensor) -> Tuple[Tensor, Tensor]:
    """Symmetric per-row int8: ``q = round(x / s)``, ``s = absmax / 127``. Returns ``(q, s[rows, 1])``."""
    if use_native(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        q = torch.empty(x2.shape, dtype=torch.int8, device=x.device)
        s = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        _native.check(lib().tpb_quant_i8_rowwise(ptr(x2), ptr(q), ptr(s), x2.shape[0], x2.shape[1],
                                                 x2.stride(0), stream_ptr()), "tpb_quant_i8_rowwise")
        return q.view(x.shape), s.view(*x.shape[:-1], 1)
    amax = x.float().abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    return torch.clamp(torch.round(x.float() / scale), -127, 127).to(torch.int8), scale


def int8_gemm(a_q: Tensor, w_q: Tensor, a_scale: Optional[Tensor] = None, w_scale: Optional[Tensor] = None,
              bias: Optional[Tensor] = None) -> Tensor:
    """``(a_q[M, K] @ w_q[N, K].T) * a_scale[m] * w_scale[n] + bias`` -> bf16, int32 accumulation."""
    M, K = a_q.shape
    N = w_q.shape[0]
    if use_native(a_q, w_q) and K % 16 == 0:
        a_q = a_q if (a_q.stride(1) == 1 and a_q.stride(0) % 16 == 0) else a_q.contiguous()
        w_q = w_q if (w_q.stride(1) == 1 and w_q.stride(0) % 16 == 0) else w_q.contiguous()
        out = torch.empty(M, N, dtype=torch.bfloat16, device=a_q.device)
        sa = None if a_scale is None else a_scale.reshape(-1).float().contiguous()
        sw = None if w_scale is None else w_scale.reshape(-1).float().contiguous()
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        _native.check(lib().tpb_gemm_i8(ptr(a_q), ptr(w_q), ptr(out), ptr(sa), ptr(sw), ptr(b), M, N, K,
                                        a_q.stride(0), w_q.stride(0), N, ptr(status_word(a_q.device)),
                                        stream_ptr()), "tpb_gemm_i8")
        return out
    acc = (a_q.to(torch.int32).cpu() @ w_q.to(torch.int32).cpu().t()).to(a_q.device).float()
    if a_scale is not None:
        acc = acc * a_scale.reshape(-1, 1).float()
    if w_scale is not None:
        acc = acc * w_scale.reshape(1, -1).float()
    if bias is not None:
        acc = acc + bias.float()
    return acc.to(torch.bfloat16)


def quantize_weight_int8(w: Tensor, group_size: int = 0) -> Tuple[Tensor, Tensor]:
    """Per-channel (``group_size = 0``) or group-wise symmetric int8. Returns ``(q[N, K], scale[N, K/g])``."""
    N, K = w.shape
    g = K if group_size <= 0 else group_size
    wf = w.float().reshape(N, K // g, g)
    amax = wf.abs().amax(dim=-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)).to(torch.bfloat16)
    q = torch.clamp(torch.round(wf / scale.float()), -127, 127).to(torch.int8)
    return q.reshape(N, K), scale.reshape(N, K // g)


def quantize_weight_int4(w: Tensor, group_size: int = 128) -> Tuple[Tensor, Tensor, Tensor]:
    """Asymmetric 4-bit group quantisation. Returns ``(packed uint8 [N, K/2], scale, zero)`` with
    ``w ~ (code - zero) * scale``; two codes per byte, low nibble first."""
    N, K = w.shape
    g = group_size
    wf = w.float().reshape(N, K // g, g)
    lo, hi = wf.amin(dim=-1, keepdim=True), wf.amax(dim=-1, keepdim=True)
    scale = ((hi - lo) / 15.0).clamp_(min=1e-8).to(torch.bfloat16)
    zero = torch.round(-lo / scale.float()).clamp_(0, 15).to(torch.bfloat16)
    code = torch.clamp(torch.round(wf / scale.float() + zero.float()), 0, 15).to(torch.uint8).reshape(N, K)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), scale.reshape(N, K // g), zero.reshape(N, K // g)


def dequantize_weight(q: Tensor, scale: Tensor, zero: Optional[Tensor] = None, bits: int = 8,
                      group_size: int = 0) -> Tensor:
    """Packed weights -> bf16 ``[N, K]``."""
    N = q.shape[0]
    K = q.shape[1] * (2 if bits == 4 else 1)
    if use_native(q, scale) and K % 8 == 0 and (group_size <= 0 or group_size % 8 == 0):
        out = torch.empty(N, K, dtype=torch.bfloat16, device=q.device)
        sc = scale.to(torch.bfloat16).contiguous()
        z = None if zero is None else zero.to(torch.bfloat16).contiguous()
        _native.check(lib().tpb_dequant_weight(ptr(q.contiguous()), ptr(sc), ptr(z), ptr(out), N, K, bits,
                                               group_size, stream_ptr()), "tpb_dequant_weight")
        return out
    g = K if group_size <= 0 else group_size
    if bits == 8:
        wf = q.float().reshape(N, K // g, g) * scale.float().reshape(N, K // g, 1)
    else:
        code = torch.stack((q & 0xF, q >> 4), dim=-1).reshape(N, K).float()
        z = zero.float().reshape(N, K // g, 1) if zero is not None else 8.0
        wf = (code.reshape(N, K // g, g) - z) * scale.float().reshape(N, K // g, 1)
    return wf.reshape(N, K).to(torch.bfloat16)


def weight_only_linear(x: Tensor, q: Tensor, scale: Tensor, zero: Optional[Tensor] = None,
                       bias: Optional[Tensor] = None, bits: int = 8, group_size: int = 0) -> Tensor:
    """``x @ dequant(q).T + bias``. Up to 16 rows of ``x`` (decode) stream the packed weights once in
    a GEMV kernel; larger inputs dequantise and use the bf16 tensor-core GEMM."""
    from .gemm import linear
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    M, N = x2.shape[0], q.shape[0]
    if (use_native(x2, q) and x2.dtype == torch.bfloat16 and M <= 16 and K % 16 == 0
            and (group_size % 16 == 0 if group_size > 0 else bits == 8)):
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        sc = scale.to(torch.bfloat16).contiguous()
        z = None if zero is None else zero.to(torch.bfloat16).contiguous()
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        _native.check(lib().tpb_wq_gemv(ptr(x2), ptr(q.contiguous()), ptr(sc), ptr(z), ptr(b), ptr(y), M, N, K,
                                        bits, group_size, x2.stride(0), N, stream_ptr()), "tpb_wq_gemv")
        return y.view(*x.shape[:-1], N)
    w = dequantize_weight(q, scale, zero, bits, group_size)
    return linear(x, w.to(x.dtype), bias)


def gemv_config(tiles: int = 0, force_simt: bool = False, version: int = 2, fold: bool = True) -> None:
    """Knobs of the weight-only GEMV for comparison runs: 16-column tiles per CTA of the warp-MMA
    kernel (0 = chosen from N), whether to force the CUDA-core kernel, which warp-MMA version runs
    (2: the default, its loop written for instruction count; 1: the first version), and whether 4-bit
    weights in groups of 128 or more take the form that applies scale and zero point per 128-k chunk
    (the default) or per weight."""
    mode = 1 if force_simt else (3 if version == 1 else (0 if fold else 4))
    lib()._lib.tpb_wq_gemv_config(int(tiles), mode)


def fp8_quantize(x: Tensor, scale: Tensor, dtype=torch.float8_e4m3fn) -> Tensor:
    """``saturate(x / scale)`` in fp8; ``scale`` is one value or one per row (last dim = row)."""
    per_row = scale.numel() > 1
    if (use_native(x) and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() % 8 == 0
            and x.shape[-1] % 8 == 0 and (not per_row or scale.numel() == x.numel() // x.shape[-1])):
        q = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        sc = scale.reshape(-1).float().contiguous()
        _native.check(lib().tpb_fp8_quant(ptr(x), ptr(sc), ptr(q), x.numel(), x.shape[-1], int(per_row),
                                          _FP8[dtype], stream_ptr()), "tpb_fp8_quant")
        return q.view(dtype)
    m = _FP8_MAX[dtype]
    return (x.float() / scale.float()).clamp_(-m, m).to(dtype)


def fp8_dequantize(q: Tensor, scale: Tensor, out_dtype=torch.bfloat16) -> Tensor:
    per_row = scale.numel() > 1
    if (use_native(q) and out_dtype == torch.bfloat16 and q.is_contiguous() and q.numel() % 8 == 0
            and q.shape[-1] % 8 == 0 and (not per_row or scale.numel() == q.numel() // q.shape[-1])):
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
        sc = scale.reshape(-1).float().contiguous()
        _native.check(lib().tpb_fp8_dequant(ptr(q.view(torch.uint8)), ptr(sc), ptr(out), q.numel(), q.shape[-1],
                                            int(per_row), _FP8[q.dtype], stream_ptr()), "tpb_fp8_dequant")
        return out
    return (q.float() * scale.float()).to(out_dtype)
