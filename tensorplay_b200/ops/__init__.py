"""Hot ops of the framework. CUDA tensors run the hand-written sm_100a kernels of
``libtpb200.so``; CPU tensors run a plain-PyTorch path that doubles as the correctness oracle."""
from ._common import DeviceWaitTimeout, check_status, status_word
from .activation import gelu, swiglu, swiglu_packed
from .attention import attention_reference, flash_attention, qkv_attention
from .decode import decode_qkv_prep, embedding, kv_append, sample, sample_reference
from .gemm import gemm, linear
from .loss import cross_entropy
from .norm import layer_norm, rms_norm
from .optim import adamw_flat_, adamw_multi_, clip_coef_, sumsq_
from .quant import (dequantize_weight, fp8_dequantize, fp8_quantize, int8_gemm, quantize_int8_rowwise,
                    quantize_weight_int4, quantize_weight_int8, weight_only_linear)
from .rope import apply_rope, rope_tables

__all__ = [
    "DeviceWaitTimeout", "check_status", "status_word", "gelu", "swiglu", "swiglu_packed", "gemm",
    "linear", "cross_entropy", "layer_norm", "rms_norm", "adamw_flat_", "adamw_multi_",
    "clip_coef_", "sumsq_", "apply_rope", "rope_tables", "attention_reference", "flash_attention",
    "qkv_attention", "embedding", "kv_append", "sample", "sample_reference", "dequantize_weight",
    "fp8_dequantize", "fp8_quantize", "int8_gemm", "quantize_int8_rowwise", "quantize_weight_int4",
    "quantize_weight_int8", "weight_only_linear",
]
