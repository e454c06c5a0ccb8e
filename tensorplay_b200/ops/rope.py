"""Rotary position embedding (NeoX half-split and GPT-J interleaved) applied in place to q and k.

Reference counterpart: p10/src/backend/cuda/transformers/AttentionRopeKernels.cu:141-272
(backward is the same rotation with the sine negated, :794-803).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native
from ._common import lib, ptr, stream_ptr, use_native


def rope_tables(max_pos: int, dim: int, theta: float = 10000.0, device=None,
                scaling: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables of shape ``[max_pos, dim // 2]``."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device) / dim))
    t = torch.arange(max_pos, dtype=torch.float64, device=device) / scaling
    ang = torch.outer(t, inv)
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def _rope_ref(x, cos, sin, pos, interleaved, sign):
    # x: [B, T, H, D]
    B, T, H, D = x.shape
    if pos is None:
        c = cos[:T].view(1, T, 1, D // 2)
        s = sin[:T].view(1, T, 1, D // 2)
    else:
        c = cos[pos].view(B, T, 1, D // 2)
        s = sin[pos].view(B, T, 1, D // 2)
    s = s * sign
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        a, b = xf[..., : D // 2], xf[..., D // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def _rope_native_(x, cos, sin, pos, interleaved, backward):
    B, T, H, D = x.shape
    if x.stride(3) != 1 or x.stride(0) != T * x.stride(1):
        raise ValueError("rope: needs [B, T, H, D] with contiguous D and uniform token stride")
    code = lib().tpb_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), ptr(pos), B * T, H, D,
                          x.stride(1), x.stride(2), T, int(interleaved), int(backward),
                          stream_ptr())
    _native.check(code, "tpb_rope")
    return x


def _rope_native_out(x, out, cos, sin, pos, interleaved, backward):
    """Rotates ``x`` (any token/head strides) into ``out``: the gather from a strided source and the rotation
    are one pass."""
    B, T, H, D = x.shape
    for t in (x, out):
        if t.stride(3) != 1 or t.stride(0) != T * t.stride(1):
            raise ValueError("rope: needs [B, T, H, D] with contiguous D and uniform token stride")
    code = lib().tpb_rope_out(x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), ptr(pos), B * T, H, D,
                              x.stride(1), x.stride(2), out.stride(1), out.stride(2), T, int(interleaved),
                              int(backward), stream_ptr())
    _native.check(code, "tpb_rope_out")
    return out


class _RopeFn(torch.autograd.Function):
    """Rotates ``x`` in place (the input buffer is consumed) and marks it dirty."""

    @staticmethod
    def forward(ctx, x, cos, sin, pos, interleaved):
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        ctx.interleaved = interleaved
        _rope_native_(x, cos, sin, pos, interleaved, False)
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        return _rotate_into_new(dy, cos, sin, pos if ctx.has_pos else None, ctx.interleaved, True), None, None, None, None


def _strided_ok(x) -> bool:
    B, T = x.shape[:2]
    return x.stride(3) == 1 and x.stride(0) == T * x.stride(1) and x.stride(1) % 8 == 0 and x.stride(2) % 8 == 0 \
        and x.data_ptr() % 16 == 0


def _rotate_into_new(x, cos, sin, pos, interleaved, backward):
    """Rotation of ``x`` into a fresh contiguous tensor; a strided ``x`` is read where it lies."""
    if not _strided_ok(x):
        x = x.contiguous()
    out = torch.empty(x.shape, device=x.device, dtype=x.dtype)
    return _rope_native_out(x, out, cos, sin, pos, interleaved, backward)


class _RopeOutFn(torch.autograd.Function):
    """Out-of-place rotation: one pass over the input, whatever its strides."""

    @staticmethod
    def forward(ctx, x, cos, sin, pos, interleaved):
        ctx.save_for_backward(cos, sin, pos if pos is not None else torch.empty(0))
        ctx.has_pos = pos is not None
        ctx.interleaved = interleaved
        return _rotate_into_new(x, cos, sin, pos, interleaved, False)

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos = ctx.saved_tensors
        return _rotate_into_new(dy, cos, sin, pos if ctx.has_pos else None, ctx.interleaved, True), None, None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
               position_ids: Optional[torch.Tensor] = None, interleaved: bool = False,
               inplace: bool = False) -> torch.Tensor:
    """Rotate ``x`` of shape ``[B, T, H, D]``; ``position_ids`` is ``[B, T]`` int64 or None."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0 and use_native(x):
        pos = None
        if position_ids is not None:
            pos = position_ids.reshape(-1).to(torch.int64).contiguous()
        needs_grad = x.requires_grad or torch.is_grad_enabled() and x.grad_fn is not None
        if not inplace:
            if needs_grad:
                return _RopeOutFn.apply(x, cos, sin, pos, interleaved)
            return _rotate_into_new(x, cos, sin, pos, interleaved, False)
        if needs_grad:
            return _RopeFn.apply(x, cos, sin, pos, interleaved)
        return _rope_native_(x, cos, sin, pos, interleaved, False)
    return _rope_ref(x, cos, sin, position_ids, interleaved, 1.0)
