"""The hot ops as PyTorch custom operators (namespace ``tpb``), so that they compose with the
dispatcher's tooling - fake tensors / meta shapes, ``torch.library.opcheck``, ``torch.export`` -
the role the reference's own dispatcher registrations play
(``TENSORPLAY_LIBRARY_IMPL(<Key>, ...){ m.impl("op", fn) }``, p10/src/backend/cuda/LinearAlgebraKernels.cu:1341-1350).

``torch.ops.tpb.rms_norm(x, w, eps)``, ``torch.ops.tpb.linear(x, w, b)``, ``torch.ops.tpb.swiglu(gate, up)``
and ``torch.ops.tpb.attention(q, k, v, causal, scale)`` run the same kernels as ``tensorplay_b200.ops``
(CUDA) or the PyTorch oracle (CPU) and carry autograd formulas that call the same backward kernels.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.library import custom_op

import importlib

# (the package re-exports functions named like its modules, so resolve the modules explicitly)
_act = importlib.import_module(__package__ + ".activation")
_attn = importlib.import_module(__package__ + ".attention")
_gemm = importlib.import_module(__package__ + ".gemm")
_norm = importlib.import_module(__package__ + ".norm")


def _via_autograd(fn, inputs, grads_out):
    """Backward of a wrapped op through the op's own autograd.Function (recomputes the forward)."""
    ins = [t.detach().requires_grad_(t.is_floating_point()) if isinstance(t, Tensor) else t for t in inputs]
    with torch.enable_grad():
        out = fn(*ins)
    tensors = [t for t in ins if isinstance(t, Tensor) and t.requires_grad]
    gs = torch.autograd.grad(out, tensors, grads_out, allow_unused=True)
    it = iter(gs)
    return tuple(next(it) if (isinstance(t, Tensor) and t.requires_grad) else None for t in ins)


@custom_op("tpb::rms_norm", mutates_args=())
def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return _norm.rms_norm(x, weight, eps).clone()


@rms_norm.register_fake
def _(x, weight, eps):
    return torch.empty_like(x)


def _rms_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1])
    ctx.eps = inputs[2]


def _rms_bwd(ctx, g):
    x, w = ctx.saved_tensors
    dx, dw = _via_autograd(lambda a, b: _norm.rms_norm(a, b, ctx.eps), (x, w), g)
    return dx, dw, None


rms_norm.register_autograd(_rms_bwd, setup_context=_rms_setup)


@custom_op("tpb::linear", mutates_args=())
def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor]) -> Tensor:
    return _gemm.linear(x, weight, bias).clone()


@linear.register_fake
def _(x, weight, bias):
    return x.new_empty(*x.shape[:-1], weight.shape[0])


def _lin_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1])
    ctx.has_bias = inputs[2] is not None


def _lin_bwd(ctx, g):
    x, w = ctx.saved_tensors
    dx, dw = _via_autograd(lambda a, b: _gemm.linear(a, b, None), (x, w), g)
    db = g.reshape(-1, g.shape[-1]).sum(0) if ctx.has_bias else None
    return dx, dw, db


linear.register_autograd(_lin_bwd, setup_context=_lin_setup)


@custom_op("tpb::swiglu", mutates_args=())
def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return _act.swiglu(gate, up).clone()


@swiglu.register_fake
def _(gate, up):
    return torch.empty_like(gate)


def _swi_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swi_bwd(ctx, g):
    a, b = ctx.saved_tensors
    return _via_autograd(_act.swiglu, (a, b), g)


swiglu.register_autograd(_swi_bwd, setup_context=_swi_setup)


@custom_op("tpb::attention", mutates_args=())
def attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, scale: float) -> Tensor:
    return _attn.flash_attention(q, k, v, causal, scale).clone()


@attention.register_fake
def _(q, k, v, causal, scale):
    return torch.empty_like(q)


def _att_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[0], inputs[1], inputs[2])
    ctx.causal, ctx.scale = inputs[3], inputs[4]


def _att_bwd(ctx, g):
    q, k, v = ctx.saved_tensors
    dq, dk, dv = _via_autograd(lambda a, b, c: _attn.flash_attention(a, b, c, ctx.causal, ctx.scale), (q, k, v), g)
    return dq, dk, dv, None, None


attention.register_autograd(_att_bwd, setup_context=_att_setup)
