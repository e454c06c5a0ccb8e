"""Model averaging for local-SGD style training: parameters are averaged over a process group every
``period`` steps instead of all-reducing gradients every step.

After tensorplay/distributed/algorithms/model_averaging (``averagers.py``: ``ModelAverager``,
``PeriodicModelAverager``; ``hierarchical_model_averager.py``: ``HierarchicalModelAverager``; ``utils.py``:
``average_parameters``, ``get_params_to_average``, ``average_parameters_or_parameter_groups``). The parameters
are packed into ONE flat buffer per dtype, averaged with one all-reduce each and copied back, so the cost of an
averaging step is one collective per dtype however many tensors the model has.
"""
from __future__ import annotations

from abc import ABC, abstractmethod
from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Union

import torch
import torch.distributed as dist


def get_params_to_average(params) -> List[torch.nn.Parameter]:
    """Parameters with gradients out of an iterable of parameters or of optimizer parameter groups."""
    out = []
    for p in params:
        if isinstance(p, torch.nn.Parameter):
            if p.grad is not None:
                out.append(p)
        elif isinstance(p, dict):
            out += [q for q in p["params"] if q.grad is not None]
        else:
            raise NotImplementedError(f"parameter input of type {type(p)} is not supported")
    return out


def average_parameters(params: Iterable[torch.Tensor], process_group=None) -> None:
    """In-place mean of every tensor over ``process_group`` (one all-reduce per dtype and device)."""
    if not dist.is_initialized():
        return
    group = process_group if process_group is not None else dist.group.WORLD
    if dist.get_rank(group) < 0:   # not a member
        return
    world = dist.get_world_size(group)
    buckets: Dict = {}
    for p in params:
        buckets.setdefault((p.dtype, p.device), []).append(p.data if isinstance(p, torch.nn.Parameter) else p)
    for (dtype, device), ts in buckets.items():
        flat = torch.cat([t.reshape(-1) for t in ts])
        if not flat.is_floating_point():
            continue
        flat.div_(world)
        if device.type == "cuda":
            torch.cuda.current_stream(device).synchronize()
        dist.all_reduce(flat, group=group)
        off = 0
        for t in ts:
            t.copy_(flat[off: off + t.numel()].view_as(t))
            off += t.numel()


def average_parameters_or_parameter_groups(params, process_group=None) -> None:
    average_parameters(get_params_to_average(params), process_group)


class ModelAverager(ABC):
    def __init__(self, process_group=None):
        self.process_group = process_group if process_group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.step = 0

    @abstractmethod
    def average_parameters(self, params):
        raise NotImplementedError


class PeriodicModelAverager(ModelAverager):
    """Averages after ``warmup_steps`` (during which gradients are still all-reduced by DDP, e.g. with
    ``post_localSGD_hook``), then every ``period`` steps."""

    def __init__(self, period: int, warmup_steps: int = 0, process_group=None):
        super().__init__(process_group)
        if warmup_steps < 0:
            raise ValueError("Arg ``warmup_steps`` must be a non-negative number.")
        if period < 1:
            raise ValueError("Arg ``period`` must be a positive value.")
        self.period, self.warmup_steps = period, warmup_steps

    def average_parameters(self, params) -> None:
        if self.step >= self.warmup_steps and (self.step - self.warmup_steps) % self.period == 0:
            average_parameters_or_parameter_groups(params, self.process_group)
        self.step += 1


class HierarchicalModelAverager(ModelAverager):
    """Several periods with growing groups: ``period_group_size_dict`` maps a period to the size of the
    sub-groups (consecutive ranks) that average at that period; the largest size must be the world size.
    At a step where several periods are due, only the largest group averages."""

    def __init__(self, period_group_size_dict: Optional["OrderedDict[int, int]"] = None, warmup_steps: int = 0,
                 process_group=None):
        super().__init__(process_group)
        if not period_group_size_dict:
            raise ValueError("Arg ``period_group_size_dict`` must not be empty.")
        periods = list(period_group_size_dict.keys())
        if periods[0] <= 0:
            raise ValueError("The minimum period in arg ``period_group_size_dict`` must be a positive value.")
        if periods != sorted(periods):
            raise ValueError("periods must be given in increasing order")
        world = dist.get_world_size(self.process_group)
        if list(period_group_size_dict.values())[-1] != world:
            raise ValueError(f"The last value in arg ``period_group_size_dict`` must be equal to the size of arg "
                             f"``process_group``: {world}")
        if warmup_steps < 0:
            raise ValueError("Arg ``warmup_steps`` must be a non-negative number.")
        self.warmup_steps = warmup_steps
        self._periods = periods
        self.period_process_group_dict: "OrderedDict[int, object]" = OrderedDict()
        rank = dist.get_rank(self.process_group)
        for period, size in period_group_size_dict.items():
            if size == world:
                self.period_process_group_dict[period] = self.process_group
                continue
            if world % size:
                raise ValueError(f"group size {size} does not divide the world size {world}")
            mine = None
            for start in range(0, world, size):   # every rank creates every sub-group, in the same order
                members = [dist.get_global_rank(self.process_group, r) if self.process_group is not dist.group.WORLD
                           else r for r in range(start, start + size)]
                g = dist.new_group(members)
                if start <= rank < start + size:
                    mine = g
            self.period_process_group_dict[period] = mine

    def _find_process_group(self):
        for period in reversed(self._periods):
            if self.step % period == 0:
                return self.period_process_group_dict[period]
        return None

    def average_parameters(self, params) -> None:
        if self.step >= self.warmup_steps:
            group = self._find_process_group()
            if group is not None:
                average_parameters_or_parameter_groups(params, group)
        self.step += 1


from . import averagers, hierarchical_model_averager, utils  # noqa: E402,F401  (the reference's sub-module paths)
