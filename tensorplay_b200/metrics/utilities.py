"""Small helpers for writing metrics: reductions over the leading dimension of list states,
class-wise reduction, and logging that speaks on rank 0 only."""
from __future__ import annotations

import logging
import os
import time
import warnings
from typing import List, Optional, Union

import torch
from torch import Tensor

_log = logging.getLogger("tensorplay_b200.metrics")


def _rank() -> int:
    if torch.distributed.is_available() and torch.distributed.is_initialized():
        return torch.distributed.get_rank()
    return int(os.environ.get("RANK", "0"))


def rank_zero_warn(message: str, *a, **kw) -> None:
    if _rank() == 0:
        warnings.warn(message, *a, **kw)


def rank_zero_info(message: str, *a, **kw) -> None:
    if _rank() == 0:
        _log.info(message, *a, **kw)


def rank_zero_debug(message: str, *a, **kw) -> None:
    if _rank() == 0:
        _log.debug(message, *a, **kw)


def dim_zero_cat(x: Union[Tensor, List[Tensor]]) -> Tensor:
    if isinstance(x, Tensor):
        return x
    x = [t.unsqueeze(0) if t.dim() == 0 else t for t in x]
    if not x:
        raise ValueError("no samples to concatenate")
    return torch.cat(x, 0)


def dim_zero_sum(x: Tensor) -> Tensor:
    return torch.sum(x, 0)


def dim_zero_mean(x: Tensor) -> Tensor:
    return torch.mean(x, 0)


def dim_zero_max(x: Tensor) -> Tensor:
    return torch.max(x, 0).values


def dim_zero_min(x: Tensor) -> Tensor:
    return torch.min(x, 0).values


def reduce(x: Tensor, reduction: Optional[str]) -> Tensor:
    if reduction in ("elementwise_mean", "mean"):
        return x.mean()
    if reduction == "sum":
        return x.sum()
    if reduction in (None, "none"):
        return x
    raise ValueError(f"unknown reduction {reduction!r}")


def class_reduce(num: Tensor, denom: Tensor, weights: Tensor, class_reduction: Optional[str] = "none") -> Tensor:
    """``num / denom`` per class reduced as "micro" (sums first), "macro", "weighted" (by
    ``weights / weights.sum()``) or "none"; 0 / 0 counts as 0."""
    if class_reduction == "micro":
        frac = num.sum() / denom.sum()
    else:
        frac = num / denom
    frac = torch.where(torch.isnan(frac), torch.zeros_like(frac), frac)
    if class_reduction in ("micro", "none", None):
        return frac
    if class_reduction == "macro":
        return frac.mean()
    if class_reduction == "weighted":
        return (frac * (weights.float() / weights.sum())).sum()
    raise ValueError(f"unknown class_reduction {class_reduction!r}")


def check_forward_full_state_property(metric_class, init_args=None, input_args=None, num_update_to_compare=(10, 100, 1000),
                                      reps: int = 5) -> None:
    """Whether ``forward`` may compute the batch value from a fresh state (one ``update`` per call)
    instead of saving and restoring the accumulated state (two): prints whether the two ways agree
    and how long each takes for the given numbers of calls."""
    init_args, input_args = init_args or {}, input_args or {}

    def run(n: int, fresh: bool):
        m = metric_class(**init_args)
        t0 = time.perf_counter()
        out = None
        for _ in range(n):
            if fresh:
                batch = metric_class(**init_args)
                batch.update(**input_args)
                out = batch.compute()
                m.update(**input_args)
            else:
                m.update(**input_args)
                out = m.compute()
        return out, time.perf_counter() - t0, m.compute()
    a, _, total_a = run(3, True)
    b, _, total_b = run(3, False)
    same_total = torch.allclose(torch.as_tensor(total_a).float(), torch.as_tensor(total_b).float())
    print(f"accumulated values agree: {same_total}; batch value needs the accumulated state: "
          f"{not torch.allclose(torch.as_tensor(a).float(), torch.as_tensor(b).float())}")
    for n in num_update_to_compare:
        tf = min(run(n, True)[1] for _ in range(reps))
        tp = min(run(n, False)[1] for _ in range(reps))
        print(f"{n} calls: fresh-state forward {tf * 1e3:.2f} ms, full-state forward {tp * 1e3:.2f} ms")


__all__ = ["check_forward_full_state_property", "class_reduce", "dim_zero_cat", "dim_zero_max", "dim_zero_mean",
           "dim_zero_min", "dim_zero_sum", "rank_zero_debug", "rank_zero_info", "rank_zero_warn", "reduce"]


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
