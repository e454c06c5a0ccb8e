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
