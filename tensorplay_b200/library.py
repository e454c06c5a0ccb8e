"""Custom-operator registration (``Library``, ``custom_op``, fake/meta kernels, autograd formulas).

The reference keeps its own dispatcher and registers ops with ``tensorplay.library``
(tensorplay/library.py); here ops are registered with PyTorch's dispatcher, which this module
re-exports, and ``register_kernel_op`` wraps one of this package's C-ABI kernels as such an op so
that it composes with ``torch.library`` tooling (fake tensors, ``opcheck``).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
from torch.library import (Library, custom_op, define, impl, impl_abstract, opcheck, register_autograd,  # noqa: F401
                           register_fake, register_kernel)

__all__ = ["Library", "custom_op", "define", "impl", "impl_abstract", "opcheck", "register_autograd",
           "register_fake", "register_kernel", "register_kernel_op"]


def register_kernel_op(name: str, fn: Callable, fake: Callable, backward: Optional[Callable] = None,
                       setup_context: Optional[Callable] = None, mutates_args=()):
    """Register ``fn`` (a Python wrapper that launches a native kernel) as the custom op ``name``
    (``"namespace::op"``) with a shape-only ``fake`` implementation and an optional autograd rule."""
    op = custom_op(name, mutates_args=mutates_args)(fn)
    op.register_fake(fake)
    if backward is not None:
        op.register_autograd(backward, setup_context=setup_context)
    return op


def __getattr__(name):
    """``CustomOpDef``, ``triton_op`` / ``wrap_triton``, ``register_vmap``, ``register_autocast``, ``infer_schema`` and ``get_kernel`` resolve to ``torch.library``."""
    import importlib
    for mod in ['torch.library']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def has_op(qualname: str) -> bool:
    """Whether ``namespace::name`` is registered with the dispatcher."""
    import torch
    ns, _, name = qualname.partition("::")
    return hasattr(getattr(torch.ops, ns, None), name.split(".")[0]) if ns and name else False


def get_op(qualname: str):
    """The ``torch.ops.namespace.name`` packet of a registered operator."""
    import torch
    ns, _, name = qualname.partition("::")
    if not has_op(qualname):
        raise KeyError(f"operator {qualname!r} is not registered")
    return getattr(getattr(torch.ops, ns), name.split(".")[0])


def tile_lang_op(*a, **k):
    raise NotImplementedError("tile-language kernels are not part of this framework: write the kernel in CUDA and "
                              "register it with register_kernel_op / custom_op, or load it with utils.cpp_jit")


wrap_tilelang = tile_lang_op
