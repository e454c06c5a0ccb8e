"""Training with uneven inputs: ranks that run out of data early keep answering the collectives of the ranks
that still train.

After tensorplay/distributed/algorithms/join.py (``JoinHook`` :21, ``Joinable`` :53, ``Join`` :119,
``notify_join_context`` :307). The protocol: every still-training rank contributes a one to a counting
all-reduce at the start of each iteration (``Join.notify_join_context``, called by the first joinable of the
context); a rank that has left its loop contributes a zero to the same all-reduce, and while the sum is positive
it runs every joinable's ``main_hook`` (which issues that iteration's collectives with neutral operands). When
the sum reaches zero, every rank runs the ``post_hook``s; the ranks that joined last are told so and can publish
the final state.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, List, NamedTuple, Optional

import torch
import torch.distributed as dist


class JoinHook:
    def main_hook(self) -> None:
        """Shadows the collectives of one training iteration."""

    def post_hook(self, is_last_joiner: bool) -> None:
        """Runs once after every rank has joined."""


class _JoinConfig(NamedTuple):
    enable: bool
    throw_on_early_termination: bool
    is_first_joinable: bool

    @staticmethod
    def disabled() -> "_JoinConfig":
        return _JoinConfig(False, False, False)


class Joinable(ABC):
    def __init__(self) -> None:
        self._join_config = _JoinConfig.disabled()

    @abstractmethod
    def join_hook(self, **kwargs) -> JoinHook: ...

    @property
    @abstractmethod
    def join_device(self) -> torch.device: ...

    @property
    @abstractmethod
    def join_process_group(self) -> Any: ...


class Join:
    def __init__(self, joinables: List[Joinable], enable: bool = True, throw_on_early_termination: bool = False,
                 **kwargs):
        if not joinables:
            raise ValueError("The join context manager requires at least one joinable")
        self._joinables = joinables
        self._enable, self._throw = enable, throw_on_early_termination
        self._hooks = [j.join_hook(**kwargs) for j in joinables]
        self._group = joinables[0].join_process_group
        self._device = joinables[0].join_device
        for j in joinables[1:]:
            if j.join_process_group is not self._group:
                raise ValueError("Using join context manager with multiple process groups")
            if j.join_device != self._device:
                raise ValueError(f"joinables on different devices: {self._device} and {j.join_device}")
        for i, j in enumerate(joinables):
            j._join_config = _JoinConfig(enable, throw_on_early_termination, i == 0)

    def __enter__(self) -> "Join":
        return self

    def _count_training_ranks(self) -> int:
        n = torch.zeros(1, device=self._device)
        dist.all_reduce(n, group=self._group)
        return int(n.item())

    def __exit__(self, etype, value, tb) -> Optional[bool]:
        if not self._enable or etype is not None:
            return None   # an exception propagates; the other ranks meet it through their own timeouts
        last = True
        while True:
            if self._count_training_ranks() == 0:
                break
            if self._throw:
                # answer the training ranks' second all-reduce with a one: they raise
                flag = torch.ones(1, device=self._device)
                dist.all_reduce(flag, group=self._group)
                raise RuntimeError(f"Rank {dist.get_rank(self._group)} exhausted all inputs.")
            last = False
            for h in self._hooks:
                h.main_hook()
        for h in self._hooks:
            h.post_hook(last)
        return None

    @staticmethod
    def notify_join_context(joinable: Joinable):
        """Called by a joinable at the start of each of its iterations. Only the first joinable of an enabled
        context communicates; returns the asynchronous work of the counting all-reduce (or None)."""
        cfg = getattr(joinable, "_join_config", None)
        if cfg is None or not cfg.enable or not cfg.is_first_joinable:
            return None
        dev, group = joinable.join_device, joinable.join_process_group
        one = torch.ones(1, device=dev)
        work = dist.all_reduce(one, group=group, async_op=True)
        if cfg.throw_on_early_termination:
            work.wait()
            flag = torch.zeros(1, device=dev)
            dist.all_reduce(flag, group=group)
            if flag.item() > 0:
                raise RuntimeError(f"Rank {dist.get_rank(group)} detected that another rank exhausted its inputs.")
        return work
