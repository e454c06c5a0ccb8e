"""Module-level quantisation workflows: ``quantize_(model, config)`` swaps the selected ``nn.Linear`` layers for a
quantised form (tensorplay/ao/quantization: ``Int8MixedPrecisionTrainingConfig``, ``Int8WeightOnlyQuantizedTrainingConfig``,
``Float8WeightOnlyConfig``, ``Float8DynamicActivationFloat8WeightConfig``, ``Int4WeightOnlyConfig`` and their layers).

What runs underneath is this framework's kernels where they exist: the tcgen05 ``kind::i8`` GEMM for int8 x int8
products (forward and both backward products of mixed-precision training), the weight-only GEMV / dequantise + bf16 GEMM
for 8- and 4-bit weights, the fp8 quantise / dequantise kernels (fp8 linear layers compute ``x @ dequant(w)^T``, as the
reference does). On CPU the same integers and the same scales go through fp32 matmuls.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
from torch import Tensor, nn

from .. import ops

__all__ = ["Int8MixedPrecisionTrainingConfig", "Int8MixedPrecisionTrainingLinear", "int8_mixed_precision_training",
           "Int8WeightOnlyQuantizedTrainingConfig", "Int8WeightOnlyQuantizedLinear", "int8_weight_only_quantized_training",
           "Int4WeightOnlyConfig", "WeightOnlyInt4Linear", "Int4WeightOnlyQuantizedLinear", "Float8WeightOnlyConfig",
           "Float8WeightOnlyInferenceConfig", "Float8WeightOnlyInferenceLinear", "float8_weight_only", "float8_weight_only_inference",
           "Float8DynamicActivationFloat8WeightConfig", "Float8DynamicActivationFloat8WeightInferenceConfig",
           "Float8DynamicActivationInferenceLinear", "float8_dynamic_activation_float8_weight",
           "float8_dynamic_activation_float8_weight_inference", "Int2WeightOnlyConfig", "int2_weight_only", "WeightOnlyInt2Linear",
           "pack_int2", "unpack_int2", "quantize_int2_weight_only", "BinaryWeightOnlyConfig", "BinaryWeightOnlyLinear"]


def _rowwise_int8(x: Tensor):
    """Per-row symmetric int8 of a 2-D tensor: ``(codes, scale [rows])``."""
    q, s = ops.quantize_int8_rowwise(x.contiguous())
    return q, s.reshape(-1).float()


def _int8_matmul(a: Tensor, b: Tensor, out_dtype) -> Tensor:
    """``a [M, K] @ b [N, K]^T`` with both operands quantised per row to int8 and an integer product."""
    a_q, a_s = _rowwise_int8(a)
    b_q, b_s = _rowwise_int8(b)
    return ops.int8_gemm(a_q, b_q, a_s, b_s).to(out_dtype)


class _Int8MixedPrecisionMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cfg):
        ctx.save_for_backward(x, weight)
        ctx.cfg = cfg
        x2 = x.reshape(-1, x.shape[-1])
        y = _int8_matmul(x2, weight, x.dtype) if cfg.output else x2 @ weight.t()
        return y.reshape(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        cfg = ctx.cfg
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        # dx = dy @ W: rows of dy against the columns of W (= rows of W^T); dW = dy^T @ x: columns against columns
        dx = _int8_matmul(dy2, weight.t().contiguous(), x.dtype) if cfg.grad_input else dy2.to(weight.dtype) @ weight
        dw = _int8_matmul(dy2.t().contiguous(), x2.t().contiguous(), weight.dtype) if cfg.grad_weight else dy2.t().to(x2.dtype) @ x2
        return dx.reshape(x.shape), dw.to(weight.dtype), None


@dataclass
class Int8MixedPrecisionTrainingConfig:
    """Which of the three products of a linear layer run as int8 x int8 with dynamic per-row scales."""
    output: bool = True
    grad_input: bool = True
    grad_weight: bool = True


int8_mixed_precision_training = Int8MixedPrecisionTrainingConfig


class Int8MixedPrecisionTrainingLinear(nn.Linear):
    """High-precision master weight, int8 tensor-core products."""

    def __init__(self, in_features, out_features, bias=True, config: Optional[Int8MixedPrecisionTrainingConfig] = None,
                 device=None, dtype=None):
        super().__init__(in_features, out_features, bias, device=device, dtype=dtype)
        self.config = config or Int8MixedPrecisionTrainingConfig()

    def forward(self, x: Tensor) -> Tensor:
        y = _Int8MixedPrecisionMatmul.apply(x, self.weight, self.config)
        return y if self.bias is None else y + self.bias


class _WeightOnlyLinear(nn.Module):
    """Frozen packed weight (8 or 4 bits, group-wise scales) and an optional bias; decode-sized inputs stream the packed
    weights once in the GEMV kernel."""

    def __init__(self, lin: nn.Linear, bits: int, group_size: int):
        super().__init__()
        self.in_features, self.out_features, self.bits, self.group_size = lin.in_features, lin.out_features, bits, group_size
        w = lin.weight.detach()
        if bits == 8:
            q, s = ops.quantize_weight_int8(w, group_size)
            z = None
        else:
            q, s, z = ops.quantize_weight_int4(w, group_size)
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s)
        self.register_buffer("zero", z)
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def forward(self, x: Tensor) -> Tensor:
        return ops.weight_only_linear(x, self.qweight, self.scale, self.zero, self.bias, self.bits, self.group_size)

    def dequantize(self) -> Tensor:
        return ops.dequantize_weight(self.qweight, self.scale, self.zero, self.bits, self.group_size)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, group_size={self.group_size}"


@dataclass
class Int8WeightOnlyQuantizedTrainingConfig:
    group_size: int = 0


int8_weight_only_quantized_training = Int8WeightOnlyQuantizedTrainingConfig


class Int8WeightOnlyQuantizedLinear(_WeightOnlyLinear):
    def __init__(self, lin: nn.Linear, group_size: int = 0):
        super().__init__(lin, 8, group_size)


@dataclass
class Int4WeightOnlyConfig:
    group_size: int = 128


class WeightOnlyInt4Linear(_WeightOnlyLinear):
    def __init__(self, lin: nn.Linear, group_size: int = 128):
        super().__init__(lin, 4, group_size)


Int4WeightOnlyQuantizedLinear = WeightOnlyInt4Linear


@dataclass
class Float8WeightOnlyConfig:
    weight_dtype: torch.dtype = torch.float8_e4m3fn


Float8WeightOnlyInferenceConfig = Float8WeightOnlyConfig
float8_weight_only = float8_weight_only_inference = Float8WeightOnlyConfig


class Float8WeightOnlyInferenceLinear(nn.Module):
    """fp8 weight with one scale per output row; ``x @ dequant(w)^T``."""

    def __init__(self, lin: nn.Linear, weight_dtype=torch.float8_e4m3fn):
        super().__init__()
        from . import choose_scale_float8
        self.in_features, self.out_features = lin.in_features, lin.out_features
        w = lin.weight.detach()
        scale = choose_scale_float8(w, weight_dtype, dim=1)
        self.register_buffer("qweight", ops.fp8_quantize(w.to(torch.bfloat16) if w.is_cuda else w, scale, weight_dtype))
        self.register_buffer("scale", scale)
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def weight(self, dtype=torch.bfloat16) -> Tensor:
        return ops.fp8_dequantize(self.qweight, self.scale, dtype)

    def forward(self, x: Tensor) -> Tensor:
        return torch.nn.functional.linear(x, self.weight(x.dtype if x.dtype != torch.float32 else torch.float32).to(x.dtype), self.bias)


@dataclass
class Float8DynamicActivationFloat8WeightConfig:
    activation_dtype: torch.dtype = torch.float8_e4m3fn
    weight_dtype: torch.dtype = torch.float8_e4m3fn


Float8DynamicActivationFloat8WeightInferenceConfig = Float8DynamicActivationFloat8WeightConfig
float8_dynamic_activation_float8_weight = float8_dynamic_activation_float8_weight_inference = Float8DynamicActivationFloat8WeightConfig


class Float8DynamicActivationInferenceLinear(Float8WeightOnlyInferenceLinear):
    """As the weight-only layer, and the activations take a round trip through fp8 with one scale per row."""

    def __init__(self, lin: nn.Linear, activation_dtype=torch.float8_e4m3fn, weight_dtype=torch.float8_e4m3fn):
        super().__init__(lin, weight_dtype)
        self.activation_dtype = activation_dtype

    def forward(self, x: Tensor) -> Tensor:
        from . import choose_scale_float8
        x2 = x.reshape(-1, x.shape[-1])
        s = choose_scale_float8(x2, self.activation_dtype, dim=1)
        xq = ops.fp8_dequantize(ops.fp8_quantize(x2, s, self.activation_dtype), s, x.dtype if x.dtype != torch.float32 else torch.float32)
        return super().forward(xq.to(x.dtype).reshape(x.shape))


# ------------------------------------------------------------------------------------------- 2-bit and 1-bit weights
def pack_int2(codes: Tensor) -> Tensor:
    """``[N, K]`` codes in 0..3 -> ``uint8 [N, ceil(K / 4)]``, lowest bits first."""
    N, K = codes.shape
    c = torch.nn.functional.pad(codes.to(torch.uint8), (0, (-K) % 4)).view(N, -1, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).contiguous()


def unpack_int2(packed: Tensor, in_features: int) -> Tensor:
    shifts = torch.tensor([0, 2, 4, 6], device=packed.device, dtype=torch.uint8)
    return ((packed.unsqueeze(-1) >> shifts) & 3).reshape(packed.shape[0], -1)[:, :in_features]


def quantize_int2_weight_only(w: Tensor, group_size: int = 64):
    """Asymmetric 2-bit group quantisation: ``(packed, scale [N, K / g], zero [N, K / g])``, ``w ~ (code - zero) * scale``."""
    N, K = w.shape
    wf = w.float().reshape(N, K // group_size, group_size)
    lo, hi = wf.amin(-1, keepdim=True), wf.amax(-1, keepdim=True)
    scale = ((hi - lo) / 3.0).clamp_min(1e-8)
    zero = torch.round(-lo / scale).clamp_(0, 3)
    codes = torch.round(wf / scale + zero).clamp_(0, 3).to(torch.uint8).reshape(N, K)
    return pack_int2(codes), scale.reshape(N, -1), zero.reshape(N, -1)


@dataclass
class Int2WeightOnlyConfig:
    group_size: int = 64


int2_weight_only = Int2WeightOnlyConfig


class WeightOnlyInt2Linear(nn.Module):
    """Two bits per weight with group-wise scale and zero point; dequantised on the fly."""

    def __init__(self, lin: nn.Linear, group_size: int = 64):
        super().__init__()
        self.in_features, self.out_features, self.group_size = lin.in_features, lin.out_features, group_size
        q, s, z = quantize_int2_weight_only(lin.weight.detach(), group_size)
        self.register_buffer("qweight", q)
        self.register_buffer("scale", s)
        self.register_buffer("zero", z)
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def dequantize(self, dtype=torch.float32) -> Tensor:
        codes = unpack_int2(self.qweight, self.in_features).float().view(self.out_features, -1, self.group_size)
        return ((codes - self.zero.unsqueeze(-1)) * self.scale.unsqueeze(-1)).reshape(self.out_features, -1).to(dtype)

    def forward(self, x: Tensor) -> Tensor:
        return torch.nn.functional.linear(x, self.dequantize(x.dtype), self.bias)


@dataclass
class BinaryWeightOnlyConfig:
    """One bit per weight: ``sign(w) * mean |w|`` per output row."""


class BinaryWeightOnlyLinear(nn.Module):
    def __init__(self, lin: nn.Linear):
        super().__init__()
        self.in_features, self.out_features = lin.in_features, lin.out_features
        w = lin.weight.detach().float()
        bits = (w >= 0).to(torch.uint8)
        K = w.shape[1]
        b = torch.nn.functional.pad(bits, (0, (-K) % 8)).view(w.shape[0], -1, 8)
        weights = (1 << torch.arange(8, dtype=torch.int32, device=w.device)).to(torch.uint8)
        self.register_buffer("qweight", (b * weights).sum(-1).to(torch.uint8))
        self.register_buffer("scale", w.abs().mean(1, keepdim=True))
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.detach().clone(), requires_grad=False)

    def dequantize(self, dtype=torch.float32) -> Tensor:
        shifts = torch.arange(8, device=self.qweight.device, dtype=torch.uint8)
        bits = ((self.qweight.unsqueeze(-1) >> shifts) & 1).reshape(self.out_features, -1)[:, : self.in_features]
        return ((bits.float() * 2 - 1) * self.scale).to(dtype)

    def forward(self, x: Tensor) -> Tensor:
        return torch.nn.functional.linear(x, self.dequantize(x.dtype), self.bias)


def _swap(model: nn.Module, make: Callable[[nn.Linear], nn.Module], filter_fn) -> nn.Module:
    for name, child in list(model.named_children()):
        if isinstance(child, nn.Linear) and type(child) is nn.Linear and (filter_fn is None or filter_fn(child, name)):
            setattr(model, name, make(child))
        else:
            _swap(child, make, filter_fn)
    return model


def quantize_(model: nn.Module, config, filter_fn: Optional[Callable[[nn.Module, str], bool]] = None) -> nn.Module:
    """In place: every plain ``nn.Linear`` that ``filter_fn(module, name)`` accepts is replaced according to ``config``
    (an instance or the class of one of the configurations of this module, or the BitNet training configuration)."""
    cfg = config() if isinstance(config, type) else config
    from .bitnet import BitNetTrainingConfig, quantize_ as _bitnet_quantize
    if isinstance(cfg, BitNetTrainingConfig):
        return _bitnet_quantize(model, cfg, filter_fn)
    if isinstance(cfg, Int8MixedPrecisionTrainingConfig):
        def make(lin):
            m = Int8MixedPrecisionTrainingLinear(lin.in_features, lin.out_features, lin.bias is not None, cfg,
                                                 device=lin.weight.device, dtype=lin.weight.dtype)
            m.weight, m.bias = lin.weight, lin.bias
            return m
    elif isinstance(cfg, Int8WeightOnlyQuantizedTrainingConfig):
        def make(lin):
            return Int8WeightOnlyQuantizedLinear(lin, cfg.group_size)
    elif isinstance(cfg, Int4WeightOnlyConfig):
        def make(lin):
            return WeightOnlyInt4Linear(lin, cfg.group_size)
    elif isinstance(cfg, Int2WeightOnlyConfig):
        def make(lin):
            return WeightOnlyInt2Linear(lin, cfg.group_size)
    elif isinstance(cfg, BinaryWeightOnlyConfig):
        def make(lin):
            return BinaryWeightOnlyLinear(lin)
    elif isinstance(cfg, Float8DynamicActivationFloat8WeightConfig):
        def make(lin):
            return Float8DynamicActivationInferenceLinear(lin, cfg.activation_dtype, cfg.weight_dtype)
    elif isinstance(cfg, Float8WeightOnlyConfig):
        def make(lin):
            return Float8WeightOnlyInferenceLinear(lin, cfg.weight_dtype)
    else:
        raise TypeError(f"quantize_: no handler for a configuration of type {type(cfg).__name__}")
    return _swap(model, make, filter_fn)
