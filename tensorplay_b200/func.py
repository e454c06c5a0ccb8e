"""``func``: PyTorch's function transforms (``vmap``, ``grad``, ``jvp``, ``functional_call`` ...) plus the names the
reference adds (tensorplay/func/__init__.py): ``chunk_vmap``, ``rearrange``, ``batch_norm_without_running_stats``."""
import torch as _torch
from torch.func import *  # noqa: F401,F403


def chunk_vmap(func, in_dims=0, out_dims=0, randomness: str = "error", chunks: int = 2):
    """``vmap`` that runs the mapped dimension in ``chunks`` pieces and concatenates: bounds the peak memory of a
    large batch of per-sample computations."""
    from torch._functorch.apis import chunk_vmap as _impl
    return _impl(func, in_dims=in_dims, out_dims=out_dims, randomness=randomness, chunks=chunks)


def rearrange(tensor, pattern: str, **axes_lengths):
    """einops-style ``rearrange`` (first-class dimensions are not needed: the einops package does it)."""
    import einops
    return einops.rearrange(tensor, pattern, **axes_lengths)


def batch_norm_without_running_stats(module: _torch.nn.Module) -> _torch.nn.Module:
    """In place: every batch-norm layer of ``module`` stops tracking running statistics (what ``vmap`` over a model
    needs, since the running buffers cannot be updated per sample)."""
    from torch.func import replace_all_batch_norm_modules_
    return replace_all_batch_norm_modules_(module)


def __getattr__(name):
    for ns_name in ("torch.func", "torch._functorch.apis", "torch._functorch.eager_transforms", "torch._functorch.functional_call"):
        import importlib
        try:
            return getattr(importlib.import_module(ns_name), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


# the reference has a package at this path: sub-module names without a file here resolve to views / PyTorch's
__path__: list = []
