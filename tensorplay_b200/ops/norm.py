"""RMSNorm / LayerNorm with fused residual add, forward and backward on sm_100a row kernels.

Reference counterparts: p10/src/backend/cuda/norm/RMSNormKernels.cu:147-486,
p10/src/backend/cuda/norm/LayerNormKernels.cu:172-1053.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native
from ._common import lib, ptr, stream_ptr, use_native


def _rows_view(x: torch.Tensor):
    H = x.shape[-1]
    if x.stride(-1) != 1:
        x = x.contiguous()
    x2 = x.reshape(-1, H)  # may copy if not viewable
    return x2, H


def _native_ok(x, w):
    return x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps, residual):
        x2, H = _rows_view(x)
        rows = x2.shape[0]
        y = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        res2 = res_out = None
        if residual is not None:
            res2 = residual.reshape(-1, H).contiguous()
            res_out = torch.empty_like(res2)
        code = lib().tpb_rmsnorm_fwd(x2.data_ptr(), ptr(res2), weight.data_ptr(), y.data_ptr(),
                                     ptr(res_out), rstd.data_ptr(), rows, H, x2.stride(0),
                                     y.stride(0), float(eps), stream_ptr())
        _native.check(code, "tpb_rmsnorm_fwd")
        xin = res_out if residual is not None else x2
        ctx.save_for_backward(xin, weight, rstd)
        ctx.shape = x.shape
        ctx.has_res = residual is not None
        ctx.w_ref = weight if hasattr(weight, "_tpb_grad_view") else None
        if residual is not None:
            return y.view(x.shape), res_out.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dres):
        xin, weight, rstd = ctx.saved_tensors
        rows, H = xin.shape
        dy2 = dy.reshape(rows, H)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dres2 = None
        if dres is not None:
            dres2 = dres.reshape(rows, H).contiguous()
        dx = torch.empty((rows, H), dtype=xin.dtype, device=xin.device)
        grid = lib().tpb_rmsnorm_bwd_grid(rows, H)
        part = torch.empty((grid, H), dtype=torch.float32, device=xin.device)
        w_ref = ctx.w_ref
        owned = w_ref is not None and w_ref._tpb_grad_view is not None
        acc = 0
        if owned:
            dw = w_ref._tpb_grad_view
            acc = int(getattr(w_ref, "_tpb_grad_written", False))
            w_ref._tpb_grad_written = True
        else:
            dw = torch.empty(H, dtype=weight.dtype, device=xin.device)
        code = lib().tpb_rmsnorm_bwd(dy2.data_ptr(), xin.data_ptr(), weight.data_ptr(),
                                     rstd.data_ptr(), ptr(dres2), dx.data_ptr(), part.data_ptr(),
                                     None, dw.data_ptr(), acc, rows, H, xin.stride(0), dy2.stride(0),
                                     dx.stride(0), stream_ptr())
        _native.check(code, "tpb_rmsnorm_bwd")
        if owned:
            dw = None
        dxv = dx.view(ctx.shape)
        return dxv, dw, None, (dxv if ctx.has_res else None)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5,
             residual: Optional[torch.Tensor] = None):
    """``y = rmsnorm(x [+ residual]) * weight``.

    With ``residual`` the sum ``x + residual`` is also returned (the new residual stream), so
    that the add, the statistics and the scale cost one pass over HBM.
    """
    if _native_ok(x, weight) and use_native(x, weight):
        y, r = _RMSNormFn.apply(x, weight, eps, residual)
        return (y, r) if residual is not None else y
    h = x if residual is None else (x + residual)
    hf = h.float()
    y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight
    return (y, h) if residual is not None else y


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x2, H = _rows_view(x)
        x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        code = lib().tpb_layernorm_fwd(x2.data_ptr(), weight.data_ptr(), ptr(bias), y.data_ptr(),
                                       mean.data_ptr(), rstd.data_ptr(), rows, H, float(eps),
                                       stream_ptr())
        _native.check(code, "tpb_layernorm_fwd")
        ctx.save_for_backward(x2, weight, mean, rstd)
        ctx.shape = x.shape
        ctx.has_bias = bias is not None
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, mean, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = dy.reshape(rows, H).contiguous()
        dx = torch.empty_like(x2)
        grid = lib().tpb_rmsnorm_bwd_grid(rows, H)
        part = torch.empty((2, grid, H), dtype=torch.float32, device=x2.device)
        dw = torch.empty(H, dtype=weight.dtype, device=x2.device)
        db = torch.empty(H, dtype=weight.dtype, device=x2.device)
        code = lib().tpb_layernorm_bwd(dy2.data_ptr(), x2.data_ptr(), weight.data_ptr(),
                                       mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                       part[0].data_ptr(), part[1].data_ptr(), None, dw.data_ptr(),
                                       None, db.data_ptr(), 0, rows, H, stream_ptr())
        _native.check(code, "tpb_layernorm_bwd")
        return dx.view(ctx.shape), dw, (db if ctx.has_bias else None), None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               eps: float = 1e-5) -> torch.Tensor:
    if _native_ok(x, weight) and use_native(x, weight):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
