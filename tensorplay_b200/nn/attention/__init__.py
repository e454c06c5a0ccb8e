"""``nn.attention``: backend selection for scaled dot-product attention, the registry of flash
implementations, and variable-length attention.

Backends of this framework: ``FLASH_ATTENTION`` = the tcgen05 flash kernels of this package
(bf16, head dim 64 / 128, causal or full, grouped heads natively); ``MATH`` = the fp32 formula
(the oracle of the kernel tests); ``EFFICIENT_ATTENTION`` / ``CUDNN_ATTENTION`` = PyTorch's library
kernels of those names. ``sdpa_kernel`` restricts which of them
``nn.functional.scaled_dot_product_attention`` may use inside the block
(tensorplay/nn/attention/__init__.py:138; registry :219-; ``varlen.py``; ``bias.py``).
"""
from __future__ import annotations

import contextlib
import enum
from typing import Callable, Dict, Iterable, List, Optional, Union

import torch

__all__ = ["SDPBackend", "sdpa_kernel", "WARN_FOR_UNFUSED_KERNELS", "register_flash_attention_impl",
           "activate_flash_attention_impl", "list_flash_attention_impls", "current_flash_attention_impl",
           "restore_flash_attention_impl", "varlen_attn", "AuxRequest", "select_backend"]

WARN_FOR_UNFUSED_KERNELS = False


class SDPBackend(enum.IntEnum):
    ERROR = -1
    MATH = 0
    FLASH_ATTENTION = 1
    EFFICIENT_ATTENTION = 2
    CUDNN_ATTENTION = 3
    OVERRIDEABLE = 4


_DEFAULT_ORDER = [SDPBackend.FLASH_ATTENTION, SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]
_enabled: List[SDPBackend] = list(_DEFAULT_ORDER)


def _cur_sdpa_kernel_backends(with_priority: bool = False) -> List[SDPBackend]:
    return list(_enabled)


@contextlib.contextmanager
def sdpa_kernel(backends: Union[List[SDPBackend], SDPBackend], set_priority: bool = False):
    """Only the given backends may serve ``scaled_dot_product_attention`` inside the block; with
    ``set_priority`` they are tried in the given order, otherwise in the default order (flash, cuDNN,
    efficient, math). The previous selection comes back on exit."""
    global _enabled
    if isinstance(backends, SDPBackend):
        backends = [backends]
    if not isinstance(backends, (list, tuple)) or not backends or not all(isinstance(b, SDPBackend) for b in backends):
        raise AssertionError("sdpa_kernel expects an SDPBackend or a non-empty list of SDPBackend")
    chosen = list(dict.fromkeys(backends))
    prev = _enabled
    _enabled = chosen if set_priority else [b for b in _DEFAULT_ORDER if b in chosen]
    try:
        yield
    finally:
        _enabled = prev


def _flash_eligible(q: torch.Tensor, k: torch.Tensor, attn_mask, dropout_p: float) -> Optional[str]:
    """None if the flash kernels can run the call, else the reason they cannot."""
    if attn_mask is not None:
        return "an explicit attention mask"
    if dropout_p != 0.0:
        return "dropout"
    if not (q.is_cuda and q.dtype == torch.bfloat16):
        return f"{q.dtype} on {q.device.type} (the kernels take bf16 on CUDA)"
    if q.dim() != 4 or q.shape[-1] not in (64, 128):
        return f"head dim {q.shape[-1]} (64 and 128 are built)"
    if q.shape[1] % k.shape[1]:
        return "query heads not a multiple of key heads"
    return None


def select_backend(q, k, v, attn_mask=None, dropout_p: float = 0.0) -> SDPBackend:
    """The first enabled backend that can run the call; raises when none can."""
    reasons = []
    for b in _enabled:
        if b == SDPBackend.FLASH_ATTENTION:
            why = _flash_eligible(q, k, attn_mask, dropout_p)
            if why is None:
                return b
            reasons.append(f"flash: {why}")
        elif b in (SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION):
            if q.is_cuda:
                return b
            reasons.append(f"{b.name.lower()}: CUDA only")
        elif b == SDPBackend.MATH:
            return b
    if WARN_FOR_UNFUSED_KERNELS:
        import warnings
        warnings.warn("no fused attention kernel for this call: " + "; ".join(reasons))
    raise RuntimeError("No available kernel for scaled_dot_product_attention among the enabled backends "
                       f"{[b.name for b in _enabled]}: " + "; ".join(reasons))


# ------------------------------------------------------------------------------------------ flash impl registry
_impls: Dict[str, Callable] = {}
_active = "tcgen05"
_previous: List[str] = []


def _builtin(q, k, v, causal, scale):
    from ...ops.attention import flash_attention
    return flash_attention(q, k, v, causal=causal, scale=scale)


_impls["tcgen05"] = _builtin


def register_flash_attention_impl(name: str, fn: Callable = None, *, register_fn: Callable = None) -> None:
    """``fn(q, k, v, causal, scale) -> o`` on ``[B, T, H, D]`` tensors becomes selectable under ``name``."""
    f = fn or register_fn
    if f is None or not callable(f):
        raise TypeError("register_flash_attention_impl needs a callable")
    _impls[name] = f


def list_flash_attention_impls() -> List[str]:
    return sorted(_impls)


def current_flash_attention_impl() -> str:
    return _active


def activate_flash_attention_impl(name: str) -> None:
    global _active
    if name not in _impls:
        raise KeyError(f"no flash attention implementation named {name!r}; registered: {list_flash_attention_impls()}")
    _previous.append(_active)
    _active = name


def restore_flash_attention_impl() -> None:
    global _active
    _active = _previous.pop() if _previous else "tcgen05"


def _flash(q, k, v, causal, scale):
    return _impls[_active](q, k, v, causal, scale)


from .varlen import AuxRequest, varlen_attn  # noqa: E402
from . import bias  # noqa: E402,F401


def __getattr__(name):
    """``flex_attention`` and the experimental sub-packages resolve to PyTorch's ``torch.nn.attention``."""
    import importlib
    if name == "omni_attention":
        # the reference's name of score-mod / block-mask attention: PyTorch's flex attention module, whose
        # ``flex_attention`` function is also reachable as ``omni_attention``
        mod = importlib.import_module("torch.nn.attention.flex_attention")
        if not hasattr(mod, "omni_attention"):
            mod.omni_attention = mod.flex_attention
        return mod
    for mod in ("torch.nn.attention", "torch.nn.attention.flex_attention", "torch.nn.attention.bias"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

from ... import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("omni_attention",))
