"""``nn.functional``: torch's functional namespace with the hot ops routed to the sm_100a kernels.

Names mirror tensorplay/nn/functional.py of the reference (``linear`` :87-112,
``scaled_dot_product_attention`` :3589-3615, ``linear_cross_entropy`` :3847-3864).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch.nn.functional import *  # noqa: F401,F403 - the long tail is torch's
import torch.nn.functional as _F

from .. import ops as _ops
from ..ops.attention import flash_attention as _flash_attention


def linear(input, weight, bias=None):
    if input.is_cuda and input.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 \
            and input.shape[-1] % 8 == 0 and weight.dim() == 2:
        return _ops.linear(input, weight, bias)
    return _F.linear(input, weight, bias)


def rms_norm(input, normalized_shape=None, weight=None, eps: Optional[float] = None):
    eps = 1e-6 if eps is None else eps
    if weight is not None and input.is_cuda and input.dtype == torch.bfloat16:
        return _ops.rms_norm(input, weight, eps)
    shape = normalized_shape if normalized_shape is not None else (input.shape[-1],)
    return _F.rms_norm(input, tuple(shape) if not isinstance(shape, int) else (shape,), weight, eps)


def layer_norm(input, normalized_shape, weight=None, bias=None, eps: float = 1e-5):
    ns = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
    if (weight is not None and len(ns) == 1 and input.is_cuda and input.dtype == torch.bfloat16
            and weight.dtype == torch.bfloat16):
        return _ops.layer_norm(input, weight, bias, eps)
    return _F.layer_norm(input, ns, weight, bias, eps)


def gelu(input, approximate: str = "none"):
    return _ops.gelu(input, approximate)


def silu_and_mul(x):
    """``silu(x[..., :d]) * x[..., d:]`` on a packed last dimension."""
    return _ops.swiglu_packed(x)


def swiglu(gate, up):
    return _ops.swiglu(gate, up)


silu_mul = swiglu
fused_swiglu = swiglu


def cross_entropy(input, target, weight=None, size_average=None, ignore_index: int = -100,
                  reduce=None, reduction: str = "mean", label_smoothing: float = 0.0):
    if (weight is None and label_smoothing == 0.0 and input.is_cuda and input.dtype == torch.bfloat16
            and target.dtype in (torch.int64, torch.int32) and input.dim() == 2):
        return _ops.cross_entropy(input, target, ignore_index, reduction)
    return _F.cross_entropy(input, target, weight=weight, ignore_index=ignore_index,
                            reduction=reduction, label_smoothing=label_smoothing)


def linear_cross_entropy(input, weight, target, bias=None, ignore_index: int = -100,
                         reduction: str = "mean"):
    """``cross_entropy(linear(input, weight, bias), target)``; on CUDA the logits gradient is
    written over the logits, so the vocabulary-sized buffer exists once."""
    logits = linear(input, weight, bias)
    return cross_entropy(logits.reshape(-1, logits.shape[-1]), target.reshape(-1),
                         ignore_index=ignore_index, reduction=reduction)


def scaled_dot_product_attention(query, key, value, attn_mask=None, dropout_p: float = 0.0,
                                 is_causal: bool = False, scale: Optional[float] = None,
                                 enable_gqa: bool = False):
    """``[B, H, T, D]`` attention. bf16 CUDA inputs without an explicit mask or dropout run on the
    tcgen05 flash kernels (grouped heads natively); anything else takes the fp32 formula or torch's
    library kernels, as ``nn.attention.sdpa_kernel`` allows."""
    from .attention import SDPBackend, _flash, select_backend
    backend = select_backend(query, key, value, attn_mask, dropout_p)
    if backend == SDPBackend.FLASH_ATTENTION:
        import math as _math
        sc = scale if scale is not None else 1.0 / _math.sqrt(query.shape[-1])
        o = _flash(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), is_causal, sc)
        return o.transpose(1, 2)
    if enable_gqa and query.shape[1] != key.shape[1]:
        g = query.shape[1] // key.shape[1]
        key = key.repeat_interleave(g, dim=1)
        value = value.repeat_interleave(g, dim=1)
    if is_causal and query.shape[-2] != key.shape[-2]:
        Tq, Tk = query.shape[-2], key.shape[-2]
        i = torch.arange(Tq, device=query.device).view(-1, 1)
        j = torch.arange(Tk, device=query.device).view(1, -1)
        attn_mask = j <= i + (Tk - Tq)
        is_causal = False
    if backend == SDPBackend.MATH or not query.is_cuda:
        tb = [torch.nn.attention.SDPBackend.MATH]
    elif backend == SDPBackend.CUDNN_ATTENTION:
        tb = [torch.nn.attention.SDPBackend.CUDNN_ATTENTION, torch.nn.attention.SDPBackend.EFFICIENT_ATTENTION,
              torch.nn.attention.SDPBackend.MATH]
    else:
        tb = [torch.nn.attention.SDPBackend.EFFICIENT_ATTENTION, torch.nn.attention.SDPBackend.MATH]
    with torch.nn.attention.sdpa_kernel(tb):
        return _F.scaled_dot_product_attention(query, key, value, attn_mask=attn_mask,
                                               dropout_p=dropout_p, is_causal=is_causal, scale=scale)


def fused_rope(x, cos, sin, position_ids=None, interleaved: bool = False):
    """Rotate ``x [B, T, H, D]`` with fp32 ``[max_pos, D/2]`` tables."""
    return _ops.apply_rope(x, cos, sin, position_ids, interleaved)
