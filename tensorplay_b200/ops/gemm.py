"""bf16 GEMM on the tcgen05 kernel, and the autograd ``linear`` built on it.

Replaces the cuBLASLt route of the reference (p10/src/backend/cuda/CudaBlasGemm.cpp:694-1052,
callers p10/src/backend/cuda/LinearAlgebraKernels.cu:1304-1350).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native
from . import _ckpt
from ._common import lib, ptr, status_word, stream_ptr, use_native


_splitk = {}


def enable_splitk(device=None, enable: bool = True) -> None:
    """Register (once per device) the fp32 workspace that lets the GEMM split the tiles of its
    last, partially filled wave along K over the idle SMs. GEMMs sharing it must run on one
    stream (they do: every op here launches on the current stream of the training loop)."""
    import ctypes as C
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    L = lib()
    raw = L._lib
    raw.tpb_gemm_splitk_workspace_bytes.restype = C.c_longlong
    if not enable:
        _splitk.pop(dev.index, None)
        L.tpb_gemm_set_splitk_workspace(None, None)
        return
    if dev.index not in _splitk:
        nbytes = raw.tpb_gemm_splitk_workspace_bytes()
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        flags = torch.zeros(1024, dtype=torch.int32, device=dev)
        _splitk[dev.index] = (ws, flags)
    ws, flags = _splitk[dev.index]
    L.tpb_gemm_set_splitk_workspace(ws.data_ptr(), flags.data_ptr())


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.stride(-1) != 1 or (t.dim() == 2 and (t.stride(0) % 8 or t.data_ptr() % 16)):
        t = t.contiguous()
    return t


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         accumulate: bool = False, out_dtype: torch.dtype = torch.bfloat16,
         alpha: float = 1.0, impl: Optional[str] = None) -> torch.Tensor:
    """``C[m, n] (+)= alpha * sum_k A(m, k) * B(n, k) (+ bias[n])``.

    ``a`` is ``[M, K]`` (``a_mn=False``) or stored transposed ``[K, M]`` (``a_mn=True``);
    ``b`` is ``[N, K]`` or stored ``[K, N]`` (``b_mn=True``). Operands are bf16, the
    accumulator fp32, ``out`` bf16 or fp32. ``impl`` pins the kernel: ``"pair"`` = the CTA-pair
    (``cta_group::2``) kernel, ``"single"`` = the one-CTA kernel, ``None`` = chosen by shape.
    """
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: reduce dims differ ({K} vs {Kb})")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if not use_native(a, b, out):
        af = (a.t() if a_mn else a).float()
        bf = (b if b_mn else b.t()).float()
        r = alpha * (af @ bf)
        if bias is not None:
            r = r + bias.float()
        if accumulate:
            r = r + out.float()
        out.copy_(r.to(out.dtype))
        return out
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm: operands must be bfloat16 on CUDA")
    a = _rowmajor(a)
    b = _rowmajor(b)
    if out.stride(-1) != 1:
        raise ValueError("gemm: out must be row-major")
    if K % 8 or a.stride(0) % 8 or b.stride(0) % 8:
        raise ValueError("gemm: leading dimensions must be multiples of 8 elements")
    st = status_word(a.device)
    fn = {None: "tpb_gemm_bf16", "pair": "tpb_gemm_bf16_pair", "single": "tpb_gemm_bf16_single"}[impl]
    code = getattr(lib(), fn)(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), ptr(bias), M, N, K,
        a.stride(0), b.stride(0), out.stride(0), int(a_mn), int(b_mn),
        int(out.dtype == torch.float32), int(bias is not None and bias.dtype == torch.float32),
        int(accumulate), float(alpha), st.data_ptr(), stream_ptr())
    _native.check(code, fn)
    if _native.flop_sinks:
        _native.add_flops("tpb.gemm", 2 * M * N * K)
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        kept = _ckpt.take()  # selective checkpointing: reuse the output of the first forward pass
        if kept is not None:
            y = kept[0]
        else:
            y = gemm(x2, weight, bias=bias, out_dtype=x2.dtype)
            _ckpt.stash(y)
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        # A training engine may own the gradient storage (a view into a flat per-unit buffer):
        # the weight-gradient GEMM then writes / accumulates there and autograd sees no grad.
        ctx.w_ref = weight if hasattr(weight, "_tpb_grad_view") else None
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, weight, b_mn=True, out_dtype=dy2.dtype).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            w_ref = ctx.w_ref
            if w_ref is not None and w_ref._tpb_grad_view is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=w_ref._tpb_grad_view,
                     accumulate=getattr(w_ref, "_tpb_grad_written", False))
                w_ref._tpb_grad_written = True
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T + bias``; on CUDA bf16 all three products run on the tcgen05 GEMM."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16) or _ckpt.active():
        return _LinearFn.apply(x, weight, bias)
    if x.is_cuda:
        # other dtypes on CUDA: cast through bf16 is not silently done; use torch's path
        return torch.nn.functional.linear(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)
