"""SwiGLU and GELU forward/backward (vectorised sm_100a kernels).

Reference counterpart: p10/src/backend/cuda/ActivationKernels.cu:420-520 (``silu_mul``,
``fused_swiglu``, ``silu_and_mul``).
"""
from __future__ import annotations

import torch

from .. import _native
from ._common import lib, stream_ptr, use_native


class _SwiGLUPackedFn(torch.autograd.Function):
    """``out = silu(gu[..., :I]) * gu[..., I:]`` for a packed ``[rows, 2I]`` input."""

    @staticmethod
    def forward(ctx, gu):
        gu2 = gu.reshape(-1, gu.shape[-1])
        if not gu2.is_contiguous():
            gu2 = gu2.contiguous()
        rows, two_i = gu2.shape
        I = two_i // 2
        out = torch.empty((rows, I), dtype=gu.dtype, device=gu.device)
        code = lib().tpb_swiglu_fwd(gu2.data_ptr(), gu2.data_ptr() + I * 2, out.data_ptr(), rows, I,
                                    two_i, stream_ptr())
        _native.check(code, "tpb_swiglu_fwd")
        ctx.save_for_backward(gu2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (gu2,) = ctx.saved_tensors
        rows, two_i = gu2.shape
        I = two_i // 2
        dy2 = dy.reshape(rows, I).contiguous()
        dgu = torch.empty_like(gu2)
        code = lib().tpb_swiglu_bwd(dy2.data_ptr(), gu2.data_ptr(), gu2.data_ptr() + I * 2,
                                    dgu.data_ptr(), dgu.data_ptr() + I * 2, rows, I, two_i, two_i,
                                    stream_ptr())
        _native.check(code, "tpb_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu_packed(gu: torch.Tensor) -> torch.Tensor:
    """SwiGLU on a packed ``[..., 2I]`` tensor holding gate then up."""
    I = gu.shape[-1] // 2
    if gu.is_cuda and gu.dtype == torch.bfloat16 and I % 8 == 0 and use_native(gu):
        return _SwiGLUPackedFn.apply(gu)
    g, u = gu[..., :I], gu[..., I:]
    return torch.nn.functional.silu(g) * u


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for separate tensors."""
    if gate.is_cuda and gate.dtype == torch.bfloat16 and gate.shape[-1] % 8 == 0 and use_native(gate):
        return swiglu_packed(torch.cat((gate, up), dim=-1))
    return torch.nn.functional.silu(gate) * up


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, approx):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        code = lib().tpb_gelu_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), int(approx), stream_ptr())
        _native.check(code, "tpb_gelu_fwd")
        ctx.save_for_backward(xc)
        ctx.approx = approx
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        code = lib().tpb_gelu_bwd(dyc.data_ptr(), xc.data_ptr(), dx.data_ptr(), xc.numel(),
                                  int(ctx.approx), stream_ptr())
        _native.check(code, "tpb_gelu_bwd")
        return dx, None


def gelu(x: torch.Tensor, approximate: str = "none") -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0 and use_native(x):
        return _GeluFn.apply(x, approximate == "tanh")
    return torch.nn.functional.gelu(x, approximate=approximate)
