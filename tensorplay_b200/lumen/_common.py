"""Shared plumbing of the attribution algorithms: input/baseline normalisation, target selection,
gradients of the selected output."""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple, Union

import torch
from torch import Tensor

TensorOrTuple = Union[Tensor, Tuple[Tensor, ...]]


def as_tuple(x: TensorOrTuple) -> Tuple[Tensor, ...]:
    return x if isinstance(x, tuple) else (x,)


def like_input(out: Tuple[Tensor, ...], ref: TensorOrTuple):
    return out if isinstance(ref, tuple) else out[0]


def make_baselines(inputs: Tuple[Tensor, ...], baselines) -> Tuple[Tensor, ...]:
    if baselines is None:
        return tuple(torch.zeros_like(i) for i in inputs)
    bs = as_tuple(baselines)
    out = []
    for i, b in zip(inputs, bs):
        if not isinstance(b, Tensor):
            b = torch.full_like(i, float(b))
        b = b.to(i.dtype)
        if b.shape != i.shape:
            b = b.expand_as(i)   # a scalar or a single example shared by the batch
        out.append(b)
    return tuple(out)


def select_target(out: Tensor, target) -> Tensor:
    """Per-example scalar of the model output: ``out[i, target]`` (int, per-example tensor or a
    tuple index for outputs with more dimensions); outputs of shape ``[B]`` / ``[B, 1]`` need none."""
    if target is None:
        if out.dim() == 1:
            return out
        if out.dim() == 2 and out.shape[1] == 1:
            return out[:, 0]
        if out.dim() == 0:
            return out.reshape(1)
        raise ValueError("the model has several outputs per example: pass target=")
    if isinstance(target, int):
        return out[:, target]
    if isinstance(target, tuple):
        return out[(slice(None),) + target]
    t = torch.as_tensor(target, device=out.device)
    if t.dim() == 0:
        return out[:, int(t)]
    reps = out.shape[0] // t.shape[0]
    if reps > 1:   # the batch was tiled (path steps, samples): tile the per-example targets alike
        t = t.repeat(reps)
    return out.gather(1, t.view(-1, 1).long())[:, 0]


def run_forward(forward_func: Callable, inputs: Tuple[Tensor, ...], target=None, additional_forward_args=None) -> Tensor:
    extra = () if additional_forward_args is None else (
        additional_forward_args if isinstance(additional_forward_args, tuple) else (additional_forward_args,))
    return select_target(forward_func(*inputs, *extra), target)


def gradients(forward_func: Callable, inputs: Tuple[Tensor, ...], target=None, additional_forward_args=None):
    with torch.enable_grad():
        ins = tuple(i.detach().requires_grad_() for i in inputs)
        out = run_forward(forward_func, ins, target, additional_forward_args)
        grads = torch.autograd.grad(out.sum(), ins, allow_unused=True)
    return tuple(torch.zeros_like(i) if g is None else g for g, i in zip(grads, ins)), out.detach()


class Attribution:
    """Base of every algorithm: wraps the model's forward function."""

    def __init__(self, forward_func: Callable):
        self.forward_func = forward_func

    def attribute(self, inputs, **kwargs):
        raise NotImplementedError

    def has_convergence_delta(self) -> bool:
        return False


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
