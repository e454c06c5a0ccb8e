"""BitNet b1.58: linear layers with ternary weights and row-wise int8 activations
(tensorplay/ao/quantization/bitnet.py: ``bitnet_linear`` :194, ``bitnet_linear_packed`` :215, ``BitNetLinear`` :244,
``BitNetTrainingLinearWeight`` :311, ``BitNetPacked2bitLinearWeight`` :435, ``BitNetTrainingConfig`` :563).

Weights: ``s_w = mean |W|``, codes ``round(W / s_w)`` clamped to {-1, 0, 1}. Activations: per row ``s_x = absmax / 127``,
codes ``round(x / s_x)`` in [-127, 127]. Output ``(x_q W_q^T) * s_x * s_w``. Training runs the same quantisers behind a
straight-through estimator (gradients as if the layer were an ordinary linear layer). On a B200 the product of the two
integer matrices is this framework's tcgen05 ``kind::i8`` GEMM with int32 accumulation - exact for integers - and both
scales go into its epilogue; elsewhere it is an fp32 matmul of the same integers. Packed weights hold four ternary codes
per byte (code + 1 in two bits, lowest bits first).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor, nn

__all__ = ["ternary_quantize", "pack_ternary", "unpack_ternary", "bitnet_linear", "bitnet_linear_packed", "BitNetLinear",
           "BitNetTrainingLinearWeight", "BitNetPacked2bitLinearWeight", "BitNetTrainingConfig", "bitnet_training"]


def ternary_quantize(weight: Tensor, eps: float = 1e-5) -> Tuple[Tensor, Tensor]:
    """``(codes int8 in {-1, 0, 1}, scale = mean |W|)``."""
    scale = weight.float().abs().mean().clamp_min(eps)
    return torch.round(weight.float() / scale).clamp_(-1, 1).to(torch.int8), scale


def _act_quantize(x: Tensor, eps: float = 1e-5) -> Tuple[Tensor, Tensor]:
    xf = x.float()
    scale = xf.abs().amax(dim=-1, keepdim=True).clamp_min(eps) / 127.0
    return torch.round(xf / scale).clamp_(-127, 127).to(torch.int8), scale


def pack_ternary(codes: Tensor) -> Tensor:
    """``[N, K]`` codes in {-1, 0, 1} -> ``uint8 [N, ceil(K / 4)]``."""
    N, K = codes.shape
    pad = (-K) % 4
    c = (codes.to(torch.int16) + 1).to(torch.uint8)
    if pad:
        c = torch.nn.functional.pad(c, (0, pad), value=1)      # the code of zero
    c = c.view(N, -1, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).contiguous()


def unpack_ternary(packed: Tensor, in_features: int) -> Tensor:
    shifts = torch.tensor([0, 2, 4, 6], device=packed.device, dtype=torch.uint8)
    c = (packed.unsqueeze(-1) >> shifts) & 3
    return (c.reshape(packed.shape[0], -1)[:, :in_features].to(torch.int8) - 1)


def _int_product(x_q: Tensor, w_q: Tensor, s_x: Tensor, s_w: Tensor, bias: Optional[Tensor], out_dtype) -> Tensor:
    """``(x_q @ w_q^T) * s_x * s_w + bias`` for integer-valued operands."""
    lead = x_q.shape[:-1]
    x2 = x_q.reshape(-1, x_q.shape[-1])
    if x2.is_cuda and x2.shape[-1] % 16 == 0:
        from ..ops import int8_gemm
        from ..ops._common import use_native
        if use_native(x2, w_q):
            sw = s_w.float().reshape(1).expand(w_q.shape[0])
            y = int8_gemm(x2.contiguous(), w_q.contiguous(), s_x.reshape(-1), sw, bias)
            return y.to(out_dtype).reshape(*lead, -1)
    y = (x2.float() @ w_q.float().t()) * s_x.reshape(-1, 1).float() * s_w.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(out_dtype).reshape(*lead, -1)


class _BitNetSTE(torch.autograd.Function):
    """Forward with quantised operands, backward of the unquantised linear layer."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        w_q, s_w = ternary_quantize(weight, eps)
        x_q, s_x = _act_quantize(x, eps)
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return _int_product(x_q, w_q, s_x, s_w, bias, x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dx = (dy.to(weight.dtype) @ weight).to(x.dtype)
        dw = dy.reshape(-1, dy.shape[-1]).t().to(x.dtype) @ x.reshape(-1, x.shape[-1])
        db = dy.reshape(-1, dy.shape[-1]).sum(0) if ctx.has_bias else None
        return dx, dw.to(weight.dtype), db, None


def bitnet_linear(input: Tensor, weight: Tensor, bias: Optional[Tensor] = None, scale: Optional[Tensor] = None,
                  eps: float = 1e-5) -> Tensor:
    """``weight`` ``[out, in]``: a float weight (quantised here, straight-through gradients), or ternary codes with
    their ``scale``."""
    if scale is not None:                      # already ternary
        x_q, s_x = _act_quantize(input, eps)
        return _int_product(x_q, weight.to(torch.int8), s_x, scale, bias, input.dtype)
    return _BitNetSTE.apply(input, weight, bias, eps)


def bitnet_linear_packed(input: Tensor, packed: Tensor, scale: Tensor, in_features: int, bias: Optional[Tensor] = None,
                         eps: float = 1e-5) -> Tensor:
    return bitnet_linear(input, unpack_ternary(packed, in_features), bias, scale, eps)


class BitNetLinear(nn.Module):
    """Float master weight, quantised at every forward (training and evaluation alike); ``pack()`` freezes it into the
    two-bit form for deployment."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)
        self.eps = 1e-5

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "BitNetLinear":
        m = cls(lin.in_features, lin.out_features, lin.bias is not None, device=lin.weight.device, dtype=lin.weight.dtype)
        with torch.no_grad():
            m.weight.copy_(lin.weight)
            if lin.bias is not None:
                m.bias.copy_(lin.bias)
        return m

    def forward(self, x: Tensor) -> Tensor:
        return bitnet_linear(x, self.weight, self.bias, eps=self.eps)

    def pack(self) -> "BitNetPacked2bitLinearWeight":
        codes, scale = ternary_quantize(self.weight.detach(), self.eps)
        return BitNetPacked2bitLinearWeight(pack_ternary(codes), scale, self.in_features)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"


class BitNetPacked2bitLinearWeight:
    """Deployment form of a BitNet weight: ``int_data`` ``uint8 [out, ceil(in / 4)]`` and the absmean ``scale``; a sixteenth
    of the bf16 bytes. ``linear(x, bias)`` applies it."""

    def __init__(self, int_data: Tensor, scale: Tensor, in_features: Optional[int] = None):
        self.int_data, self.scale = int_data, scale
        self.in_features = int(in_features) if in_features is not None else int_data.shape[1] * 4

    @property
    def shape(self) -> torch.Size:
        return torch.Size((self.int_data.shape[0], self.in_features))

    def dequantize(self, dtype=torch.float32) -> Tensor:
        return (unpack_ternary(self.int_data, self.in_features).float() * self.scale.float()).to(dtype)

    def linear(self, x: Tensor, bias: Optional[Tensor] = None) -> Tensor:
        return bitnet_linear_packed(x, self.int_data, self.scale, self.in_features, bias)

    def to(self, *args, **kwargs) -> "BitNetPacked2bitLinearWeight":
        return BitNetPacked2bitLinearWeight(self.int_data.to(*args, **kwargs), self.scale.to(*args, **kwargs), self.in_features)

    def nbytes(self) -> int:
        return self.int_data.numel() + self.scale.numel() * self.scale.element_size()


class BitNetTrainingLinearWeight(nn.Parameter):
    """Marker type of a weight that trains under BitNet quantisation: ``nn.functional.linear`` calls that receive it go
    through the straight-through estimator."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.nn.functional.linear and len(args) >= 2 and isinstance(args[1], cls):
            x, w = args[0], args[1]
            bias = args[2] if len(args) > 2 else kwargs.get("bias")
            with torch._C.DisableTorchFunctionSubclass():
                return bitnet_linear(x, w.as_subclass(torch.Tensor), bias)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)


class BitNetTrainingConfig:
    """Configuration marker of :func:`quantize_`: every ``nn.Linear`` that the filter accepts gets a BitNet training weight."""


bitnet_training = BitNetTrainingConfig


def quantize_(model: nn.Module, config=None, filter_fn=None) -> nn.Module:
    """In place: the weights of the selected ``nn.Linear`` layers become :class:`BitNetTrainingLinearWeight`."""
    if config is not None and not isinstance(config, BitNetTrainingConfig) and config is not BitNetTrainingConfig:
        raise TypeError("quantize_: only the BitNet training configuration is handled here")
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear) and (filter_fn is None or filter_fn(m, name)):
            m.weight = BitNetTrainingLinearWeight(m.weight.data, requires_grad=m.weight.requires_grad)
    return model
