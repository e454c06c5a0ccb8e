"""Collective spellings of the reference that PyTorch does not have under these names
(tensorplay/distributed/distributed_core.py: ``record_comm`` :575, ``set_timeout`` :716, ``register_device_backend``
:783, ``gather_single`` :1595, ``gather_into_tensor`` :1666, ``all_gather_single_coalesced`` :2081,
``reduce_scatter_single_coalesced`` :2254, ``reduce_scatter_coalesced`` :2471). The coalesced forms pack their
tensors into ONE flat buffer per dtype and issue one collective for it: launch latency, not link count, is what a
list of small tensors costs on NVSwitch."""
from __future__ import annotations

import contextlib
import threading
from datetime import timedelta
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist
from torch._C._distributed_c10d import AllgatherOptions  # noqa: F401

SHRINK_DEFAULT = 0x00
SHRINK_ABORT = 0x01

_comm_names = threading.local()
_device_backends: Dict[str, Callable[[Any], Any]] = {}


@contextlib.contextmanager
def record_comm(name: str):
    """Names the communication issued inside the block: the name is pushed as a profiler range (NVTX on CUDA) and
    is readable through ``current_comm_name()`` by hooks and loggers."""
    if not isinstance(name, str):
        raise TypeError("communication profiling name must be a string")
    stack = getattr(_comm_names, "stack", None)
    if stack is None:
        stack = _comm_names.stack = []
    stack.append(name)
    with torch.profiler.record_function(f"comm::{name}"):
        try:
            yield
        finally:
            stack.pop()


def current_comm_name() -> Optional[str]:
    stack = getattr(_comm_names, "stack", None)
    return stack[-1] if stack else None


def set_timeout(timeout: timedelta, group=None) -> None:
    """Timeout of the operations issued on ``group`` from now on."""
    pg = group if group is not None else dist.group.WORLD
    if not isinstance(timeout, timedelta):
        raise TypeError("timeout must be a datetime.timedelta")
    for dev in ("cuda", "cpu"):
        try:
            pg._get_backend(torch.device(dev))._set_default_timeout(timeout)
        except Exception:
            pass
    if hasattr(pg, "_set_default_timeout"):
        try:
            pg._set_default_timeout(timeout)
        except Exception:
            pass


def register_device_backend(name: str, factory: Callable[[Any], Any]) -> None:
    """Records ``factory(process_group) -> provider`` as the collective provider of the device backend ``name``;
    ``device_backend_factory(name)`` returns it. (Making ``name`` a backend of ``init_process_group`` takes a creator
    that builds a process group from a store: ``Backend.register_backend``.)"""
    if not callable(factory):
        raise TypeError("device backend factory must be callable")
    _device_backends[str(name).lower()] = factory


def device_backend_factory(name: str) -> Optional[Callable[[Any], Any]]:
    return _device_backends.get(str(name).lower())


def _group_dst(group, dst: Optional[int], group_dst: Optional[int]) -> int:
    if dst is not None and group_dst is not None:
        raise ValueError("pass dst or group_dst, not both")
    if group_dst is not None:
        return dist.get_global_rank(group, group_dst) if group is not None else group_dst
    return 0 if dst is None else dst


def gather_single(tensor: torch.Tensor, gather_tensor: Optional[torch.Tensor] = None, dst: Optional[int] = None,
                  group=None, async_op: bool = False, group_dst: Optional[int] = None):
    """Gathers one tensor per rank into ONE tensor on ``dst`` (``[world * n, ...]`` along dim 0, or any tensor of
    ``world`` times the elements)."""
    dst = _group_dst(group, dst, group_dst)
    world = dist.get_world_size(group)
    on_dst = dist.get_rank() == dst
    if on_dst:
        if gather_tensor is None:
            raise ValueError("gather_tensor is required on the destination rank")
        if gather_tensor.numel() != world * tensor.numel():
            raise ValueError("gather_tensor must hold world_size times the elements of tensor")
        flat = gather_tensor.view(-1) if gather_tensor.is_contiguous() else torch.empty(
            world * tensor.numel(), dtype=tensor.dtype, device=tensor.device)
        parts = list(flat.view(world, -1).unbind(0))
    else:
        flat, parts = None, None
    work = dist.gather(tensor.contiguous().view(-1), parts, dst=dst, group=group, async_op=async_op)
    if on_dst and flat.data_ptr() != gather_tensor.data_ptr():
        if async_op:
            work.wait()
        gather_tensor.copy_(flat.view_as(gather_tensor))
    return work


def gather_into_tensor(tensor, gather_tensor=None, dst=None, group=None, async_op=False, group_dst=None):
    return gather_single(tensor, gather_tensor, dst, group, async_op, group_dst=group_dst)


class _Works:
    """The works of a coalesced call behave as one."""

    def __init__(self, works, after: Optional[Callable[[], None]] = None):
        self.works, self.after = [w for w in works if w is not None], after

    def wait(self, timeout=None) -> bool:
        for w in self.works:
            w.wait()
        if self.after is not None:
            self.after()
            self.after = None
        return True

    def is_completed(self) -> bool:
        return all(w.is_completed() for w in self.works)


def _by_dtype(tensors: List[torch.Tensor]) -> Dict[Any, List[int]]:
    out: Dict[Any, List[int]] = {}
    for i, t in enumerate(tensors):
        out.setdefault((t.dtype, t.device), []).append(i)
    return out


def all_gather_single_coalesced(output_tensor_list: List[torch.Tensor], input_tensor_list: List[torch.Tensor],
                                group=None, async_op: bool = False):
    """``output[i]`` (``world`` times the elements of ``input[i]``, rank-major) for every ``i``, with one all-gather
    per dtype: the inputs are packed into one buffer, gathered, and unpacked."""
    if len(output_tensor_list) != len(input_tensor_list):
        raise ValueError("output_tensor_list and input_tensor_list must have the same length")
    if not input_tensor_list:
        raise ValueError("all_gather_single_coalesced requires a non-empty tensor list")
    world = dist.get_world_size(group)
    works, unpack = [], []
    for (_dtype, _dev), idx in _by_dtype(input_tensor_list).items():
        sizes = [input_tensor_list[i].numel() for i in idx]
        packed = torch.cat([input_tensor_list[i].reshape(-1) for i in idx])
        gathered = torch.empty(world * packed.numel(), dtype=packed.dtype, device=packed.device)
        works.append(dist.all_gather_into_tensor(gathered, packed, group=group, async_op=async_op))

        def fill(idx=idx, sizes=sizes, gathered=gathered, n=packed.numel()):
            rows = gathered.view(world, n)
            off = 0
            for i, sz in zip(idx, sizes):
                out = output_tensor_list[i]
                if out.numel() != world * sz:
                    raise ValueError(f"output {i} must hold world_size times the elements of input {i}")
                out.copy_(rows[:, off: off + sz].reshape(out.shape))
                off += sz
        unpack.append(fill)

    def after():
        for f in unpack:
            f()
    if async_op:
        return _Works(works, after)
    after()
    return None


def reduce_scatter_single_coalesced(output_tensor_list: List[torch.Tensor], input_tensor_list: List[torch.Tensor],
                                    op=dist.ReduceOp.SUM, group=None, async_op: bool = False):
    """``output[i]`` = this rank's slice of the reduction of ``input[i]`` (flattened, ``world`` equal slices), one
    reduce-scatter per dtype over a buffer packed slice-major."""
    if len(output_tensor_list) != len(input_tensor_list):
        raise ValueError("output_tensor_list and input_tensor_list must have the same length")
    if not input_tensor_list:
        raise ValueError("reduce_scatter_single_coalesced requires a non-empty tensor list")
    world = dist.get_world_size(group)
    works, unpack = [], []
    for (_dtype, _dev), idx in _by_dtype(input_tensor_list).items():
        for i in idx:
            if input_tensor_list[i].numel() != world * output_tensor_list[i].numel():
                raise ValueError(f"input {i} must hold world_size times the elements of output {i}")
        sizes = [output_tensor_list[i].numel() for i in idx]
        # rank-major packing: row r holds every tensor's slice r, so that one reduce-scatter hands rank r its row
        packed = torch.cat([input_tensor_list[i].reshape(world, -1) for i in idx], dim=1).contiguous()
        mine = torch.empty(packed.shape[1], dtype=packed.dtype, device=packed.device)
        works.append(dist.reduce_scatter_tensor(mine, packed.view(-1), op=op, group=group, async_op=async_op))

        def fill(idx=idx, sizes=sizes, mine=mine):
            off = 0
            for i, sz in zip(idx, sizes):
                output_tensor_list[i].copy_(mine[off: off + sz].view_as(output_tensor_list[i]))
                off += sz
        unpack.append(fill)

    def after():
        for f in unpack:
            f()
    if async_op:
        return _Works(works, after)
    after()
    return None


def reduce_scatter_coalesced(output_tensor_list: List[torch.Tensor], input_tensor_lists: List[List[torch.Tensor]],
                             op=dist.ReduceOp.SUM, group=None, async_op: bool = False):
    """``output[i]`` = reduction over ranks of ``input_tensor_lists[i][rank]``; all of them in one packed
    reduce-scatter per dtype."""
    if len(output_tensor_list) != len(input_tensor_lists):
        raise ValueError("output_tensor_list and input_tensor_lists must have the same length")
    world = dist.get_world_size(group)
    flat_inputs = []
    for i, lst in enumerate(input_tensor_lists):
        if len(lst) != world:
            raise ValueError(f"input_tensor_lists[{i}] must have one tensor per rank")
        flat_inputs.append(torch.stack([t.reshape(-1) for t in lst]))
    return reduce_scatter_single_coalesced(output_tensor_list, flat_inputs, op=op, group=group, async_op=async_op)
