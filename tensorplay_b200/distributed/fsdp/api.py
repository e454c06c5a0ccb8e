"""``fully_shard`` on flat per-unit buffers.

Every call of ``fully_shard`` makes one *unit*: the parameters the call owns are sharded on dim 0
(ceil chunks with padding, tensorplay/distributed/fsdp/_fully_shard/_fsdp_param.py:284-374) and the
local chunks of all of them live side by side in ONE flat shard. A unit therefore costs one
all-gather and one reduce-scatter, whatever its number of parameters (the reference's
``foreach_all_gather`` / ``foreach_reduce``, _fsdp_collectives.py:337-623): the gathered
``[world, S]`` buffer is copied out into per-parameter full tensors, the full gradients are copied
into a ``[world, S]`` buffer, reduced, and the result is added to the flat gradient that the sharded
parameters' ``.grad`` are views of.

On a 2-D mesh (replicate, shard) the reduced shard is also all-reduced over the replicate
dimension (hybrid sharding). ``MixedPrecisionPolicy``, ``CPUOffloadPolicy``, custom all-gather /
reduce-scatter objects (``Comm``), the all-reduce hook and the gradient-sync / reshard switches of
``FSDPModule`` are honoured; arguments that are not implemented raise instead of being ignored.
The sharded training engine for transformer stacks (peer-memory kernels, optimizer in backward) is
``tensorplay_b200.parallel.FSDPEngine``.
"""
from __future__ import annotations

import contextlib
import enum
from abc import ABC, abstractmethod
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple, Union

import torch
import torch.distributed as dist
from torch import nn


# ------------------------------------------------------------------------------------------ policies
@dataclass
class MixedPrecisionPolicy:
    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: Optional[torch.dtype] = None
    output_dtype: Optional[torch.dtype] = None
    cast_forward_inputs: bool = True


@dataclass
class OffloadPolicy:
    pass


@dataclass
class CPUOffloadPolicy(OffloadPolicy):
    """Sharded parameters, their gradients (and so the optimizer state) live in host memory; a unit's
    shard is copied to the device for its all-gather and its reduced gradient back to the host."""
    pin_memory: bool = True


@dataclass
class DataParallelMeshDims:
    """Names of the mesh dimensions used for sharding and (hybrid) replication."""
    shard: Union[str, Tuple[str, ...], None] = None
    replicate: Union[str, Tuple[str, ...], None] = None


class ShardingStrategy(enum.Enum):
    FULL_SHARD = 1
    SHARD_GRAD_OP = 2
    NO_SHARD = 3
    HYBRID_SHARD = 4
    _HYBRID_SHARD_ZERO2 = 5


@dataclass
class MixedPrecision:
    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: Optional[torch.dtype] = None
    buffer_dtype: Optional[torch.dtype] = None


@dataclass
class CPUOffload:
    offload_params: bool = False


class BackwardPrefetch(enum.Enum):
    BACKWARD_PRE = 1
    BACKWARD_POST = 2


# ------------------------------------------------------------------------------------------ comm plug points
class Comm(ABC):
    """Buffer provider of a custom collective (tensorplay/distributed/fsdp/_fully_shard/_fsdp_api.py:28-44)."""

    @abstractmethod
    def allocate(self, size: Sequence[int], *, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.empty(tuple(size), dtype=dtype, device=device)


class AllGather(Comm):
    @abstractmethod
    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group, async_op: bool = False):
        raise NotImplementedError


class ReduceScatter(Comm):
    @abstractmethod
    def __call__(self, output_tensor: torch.Tensor, input_tensor: torch.Tensor, group, op, async_op: bool = False):
        raise NotImplementedError


class _DefaultAllGather(AllGather):
    def allocate(self, size, *, dtype, device):
        return torch.empty(tuple(size), dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, async_op=False):
        if group is None and not dist.is_initialized():
            output_tensor.copy_(input_tensor)
            return None
        return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group, async_op=async_op)


class _DefaultReduceScatter(ReduceScatter):
    def allocate(self, size, *, dtype, device):
        return torch.empty(tuple(size), dtype=dtype, device=device)

    def __call__(self, output_tensor, input_tensor, group, op=dist.ReduceOp.SUM, async_op=False):
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        if world == 1:
            output_tensor.copy_(input_tensor.view(-1)[: output_tensor.numel()].view_as(output_tensor))
            return None
        if dist.get_backend(group) == "gloo":
            # gloo has no reduce-scatter: all-reduce, keep the own slice
            dist.all_reduce(input_tensor, op=op, group=group)
            r = dist.get_rank(group)
            n = output_tensor.numel()
            output_tensor.copy_(input_tensor.view(-1)[r * n: (r + 1) * n].view_as(output_tensor))
            return None
        return dist.reduce_scatter_tensor(output_tensor, input_tensor, op=op, group=group, async_op=async_op)


# ------------------------------------------------------------------------------------------ one parameter
class _ShardedParam:
    """One parameter of a unit: where its padded local chunk sits in the flat shard and how the full
    tensor is rebuilt from the gathered buffer."""

    def __init__(self, module: nn.Module, name: str, param: nn.Parameter, world: int, rank: int):
        self.module, self.name = module, name
        self.full_shape = tuple(param.shape)
        self.orig_dtype = param.dtype
        self.requires_grad = param.requires_grad
        n0 = self.full_shape[0] if self.full_shape else 1
        self.n0 = n0
        self.rest = tuple(self.full_shape[1:])
        self.rest_numel = 1
        for d in self.rest:
            self.rest_numel *= d
        self.chunk = (n0 + world - 1) // world                      # rows per rank (the last ranks may hold fewer / none)
        self.local_rows = max(0, min(self.chunk, n0 - rank * self.chunk))
        self.seg = self.chunk * self.rest_numel                     # elements of this parameter in every rank's flat shard
        self.offset = 0                                             # set by the unit
        self.sharded: Optional[nn.Parameter] = None
        self.unsharded: Optional[torch.Tensor] = None
        self.kept: Optional[torch.Tensor] = None

    def local_view(self, flat: torch.Tensor) -> torch.Tensor:
        """This rank's rows as a view of the flat shard (a 0-dim parameter is treated as shape (1,):
        rank 0 holds it, the other ranks an empty piece)."""
        n = self.local_rows * self.rest_numel
        return flat[self.offset: self.offset + n].view((self.local_rows,) + self.rest)

    def bind_sharded(self) -> None:
        self.module.__dict__.pop(self.name, None)
        self.module._parameters[self.name] = self.sharded
        self.unsharded = None

    def bind_unsharded(self, full: torch.Tensor) -> None:
        self.unsharded = full
        # plain tensor attribute (not a registered parameter) for the duration of the compute
        self.module._parameters.pop(self.name, None)
        object.__setattr__(self.module, self.name, full)


# ------------------------------------------------------------------------------------------ one unit
class _FSDPState:
    def __init__(self, module: nn.Module, infos: List[_ShardedParam], originals: List[nn.Parameter], shard_group,
                 replicate_group, mp: MixedPrecisionPolicy, offload: OffloadPolicy, reshard_after_forward: bool):
        self.module, self.params = module, infos
        self.group, self.replicate_group = shard_group, replicate_group
        init = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(shard_group) if init else 1
        self.rank = dist.get_rank(shard_group) if init else 0
        self.rep_world = dist.get_world_size(replicate_group) if (init and replicate_group is not None) else 1
        self.mp = mp
        self.cpu_offload = isinstance(offload, CPUOffloadPolicy)
        self.reshard_after_forward = reshard_after_forward
        self.reshard_after_backward = True
        self.reduce_grads = True
        self.requires_all_reduce = True
        self.is_last_backward = True
        self.unshard_in_backward = True
        self.divide: Optional[float] = None          # gradient divide factor (default: the data-parallel size)
        self.force_sum = False
        self.is_unsharded = False
        self.fwd_prefetch: list = []
        self.bwd_prefetch: list = []
        self.all_gather_comm: AllGather = _DefaultAllGather()
        self.reduce_scatter_comm: ReduceScatter = _DefaultReduceScatter()
        self.all_reduce_hook: Optional[Callable[[torch.Tensor], None]] = None
        self.all_reduce_hook_stream = None
        self.post_optim_event = None
        self.unreduced: Optional[torch.Tensor] = None   # [world, S] sum of full gradients while sync is off
        self.partial: Optional[torch.Tensor] = None     # [S] reduce-scattered, not yet all-reduced (HSDP, all-reduce off)
        self.comm_ctx: dict = {}
        self.collective_counts = {"all_gather": 0, "reduce_scatter": 0, "all_reduce": 0}
        # ---- flat layout: segments aligned to 8 elements so that any dtype's slices stay 16-byte aligned
        off = 0
        for p in infos:
            p.offset = off
            off += (p.seg + 7) // 8 * 8
        self.S = max(off, 8)
        first = originals[0] if originals else None
        self.device = first.device if first is not None else torch.device("cpu")
        self.orig_dtype = first.dtype if first is not None else torch.float32
        if any(o.dtype != self.orig_dtype for o in originals):
            raise ValueError("fully_shard: the parameters of one unit must share a dtype "
                             "(shard modules of different dtypes separately)")
        host = torch.device("cpu") if self.cpu_offload else self.device
        self.flat_shard = torch.zeros(self.S, dtype=self.orig_dtype, device=host)
        if self.cpu_offload and getattr(offload, "pin_memory", False) and torch.cuda.is_available():
            self.flat_shard = self.flat_shard.pin_memory()
        self.flat_grad: Optional[torch.Tensor] = None
        for p, orig in zip(infos, originals):
            data = orig.data if orig.dim() else orig.data.reshape(1)
            if p.local_rows:
                rows = data[self.rank * p.chunk: self.rank * p.chunk + p.local_rows]
                self.flat_shard[p.offset: p.offset + rows.numel()].copy_(rows.reshape(-1))
            p.sharded = nn.Parameter(p.local_view(self.flat_shard), requires_grad=orig.requires_grad)
            p.sharded._fsdp_info = p
            p.sharded._fsdp_state = self
            p.bind_sharded()

    # ---- navigation
    def tree(self, recurse: bool):
        yield self
        if recurse:
            seen = {id(self)}
            for m in self.module.modules():
                st = getattr(m, "_fsdp_state", None)
                if st is not None and id(st) not in seen:
                    seen.add(id(st))
                    yield st

    # ---- unshard / reshard
    def unshard(self) -> None:
        if self.is_unsharded or not self.params:
            self.is_unsharded = True
            return
        if self.post_optim_event is not None:
            # the optimizer step ran on another stream: its event orders the gather after it
            torch.cuda.current_stream().wait_event(self.post_optim_event)
            self.post_optim_event = None
        dt = self.mp.param_dtype or self.orig_dtype
        src = self.flat_shard
        if self.cpu_offload:
            src = src.to(self.device, non_blocking=True)
        if src.dtype != dt:
            src = src.to(dt)
        ag = self.all_gather_comm
        out = ag.allocate((self.world * self.S,), dtype=dt, device=src.device)
        work = ag(out, src.contiguous(), self.group)
        if work is not None and hasattr(work, "wait"):
            work.wait()
        self.collective_counts["all_gather"] += 1
        out2 = out.view(self.world, self.S)
        total = sum(self.world * p.seg for p in self.params)
        full_flat = torch.empty(total, dtype=dt, device=out.device)
        dsts, srcs, pos = [], [], 0
        for p in self.params:
            n = self.world * p.seg
            dsts.append(full_flat[pos: pos + n].view(self.world, p.seg))
            srcs.append(out2[:, p.offset: p.offset + p.seg])
            pos += n
        torch._foreach_copy_(dsts, srcs)
        for p, d in zip(self.params, dsts):
            full = d.view(-1)[: p.n0 * p.rest_numel].view(p.full_shape)
            p.bind_unsharded(full.requires_grad_(p.requires_grad))
        self.is_unsharded = True

    def reshard(self) -> None:
        if self.is_unsharded:
            for p in self.params:
                p.bind_sharded()
            self.is_unsharded = False

    # ---- hooks
    def pre_forward(self, module, args, kwargs):
        self.unshard()
        for m in self.fwd_prefetch:
            m._fsdp_state.unshard()
        if self.mp.cast_forward_inputs and self.mp.param_dtype is not None:
            dt = self.mp.param_dtype
            cast = lambda t: t.to(dt) if isinstance(t, torch.Tensor) and t.is_floating_point() and t.dtype != dt else t  # noqa: E731
            args = tuple(cast(a) for a in args)
            kwargs = {k: cast(v) for k, v in kwargs.items()}
        return args, kwargs

    def post_forward(self, module, args, output):
        need_bwd = torch.is_grad_enabled() and any(p.requires_grad for p in self.params)
        if need_bwd:
            _register_post_backward(self)
        if self.reshard_after_forward:
            if need_bwd:
                # the autograd graph keeps the gathered tensors alive; the module goes back to its
                # sharded parameters now and the gradients are read from those tensors in backward
                for p in self.params:
                    p.kept = p.unsharded
            self.reshard()
        if self.mp.output_dtype is not None:
            dt = self.mp.output_dtype
            conv = lambda t: t.to(dt) if isinstance(t, torch.Tensor) and t.is_floating_point() else t  # noqa: E731
            output = type(output)(conv(o) for o in output) if isinstance(output, (tuple, list)) else conv(output)
        return output

    def _divide_factor(self) -> float:
        return float(self.divide) if self.divide is not None else float(self.world * self.rep_world)

    def post_backward(self, fulls: Optional[list] = None) -> None:
        """``fulls``: the gathered tensors of the forward whose backward just finished. Several
        forwards may precede the first backward (pipeline micro-batches), each with its own gathered
        copies, so the gradients are read from the copies that forward used."""
        grads = []
        for i, p in enumerate(self.params):
            full = fulls[i] if fulls is not None else (p.unsharded if p.unsharded is not None else p.kept)
            g = full.grad if full is not None else None
            if full is not None:
                full.grad = None
            if p.kept is full:
                p.kept = None
            grads.append(g)
        if any(g is not None for g in grads):
            self._reduce(grads)
        if self.reshard_after_backward:
            self.reshard()

    def _reduce(self, grads: List[Optional[torch.Tensor]]) -> None:
        dev = next(g for g in grads if g is not None).device
        rd = self.mp.reduce_dtype or next(g for g in grads if g is not None).dtype
        needs_zero = any(g is None or self.world * p.chunk != p.n0 or p.seg % 8 for g, p in zip(grads, self.params))
        alloc = torch.zeros if needs_zero else torch.empty
        flat_in = alloc((self.world, self.S), dtype=rd, device=dev)
        dsts, srcs = [], []
        for g, p in zip(grads, self.params):
            if g is None:
                continue
            g2 = g.reshape(p.n0, p.rest_numel)
            full_rows = p.n0 // p.chunk if p.chunk else 0
            if full_rows:
                dsts.append(flat_in[:full_rows, p.offset: p.offset + p.seg].view(full_rows, p.chunk, p.rest_numel))
                srcs.append(g2[: full_rows * p.chunk].view(full_rows, p.chunk, p.rest_numel))
            tail = p.n0 - full_rows * p.chunk
            if tail:
                dsts.append(flat_in[full_rows, p.offset: p.offset + tail * p.rest_numel].view(tail, p.rest_numel))
                srcs.append(g2[full_rows * p.chunk:])
        srcs = [s if s.dtype == rd else s.to(rd) for s in srcs]
        torch._foreach_copy_(dsts, srcs)
        if not self.reduce_grads:
            # gradient synchronisation is off (accumulation steps): keep the full-size sum locally
            self.unreduced = flat_in if self.unreduced is None else self.unreduced.add_(flat_in)
            return
        if self.unreduced is not None:
            flat_in.add_(self.unreduced)
            self.unreduced = None
        rs = self.reduce_scatter_comm
        out = rs.allocate((self.S,), dtype=rd, device=dev)
        work = rs(out, flat_in, self.group, op=dist.ReduceOp.SUM)
        if work is not None and hasattr(work, "wait"):
            work.wait()
        self.collective_counts["reduce_scatter"] += 1
        if self.replicate_group is not None:
            if not self.requires_all_reduce:
                self.partial = out if self.partial is None else self.partial.add_(out)
                return
            if self.partial is not None:
                out.add_(self.partial)
                self.partial = None
            dist.all_reduce(out, group=self.replicate_group)
            self.collective_counts["all_reduce"] += 1
        if self.all_reduce_hook is not None:
            if self.all_reduce_hook_stream is not None:
                self.all_reduce_hook_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.all_reduce_hook_stream):
                    self.all_reduce_hook(out)
                torch.cuda.current_stream().wait_stream(self.all_reduce_hook_stream)
            else:
                self.all_reduce_hook(out)
        if not self.force_sum or self.divide is not None:
            f = self._divide_factor()
            if f != 1.0:
                out.div_(f)
        red = out.to(self.orig_dtype)
        if self.cpu_offload:
            red = red.to("cpu", non_blocking=False)
        if self.flat_grad is None or any(p.sharded.grad is None for p in self.params if p.requires_grad):
            self.flat_grad = red.clone() if red.data_ptr() == out.data_ptr() else red
            for p in self.params:
                if p.requires_grad:
                    n = p.local_rows * p.rest_numel
                    v = self.flat_grad[p.offset: p.offset + n]
                    p.sharded.grad = v.view(p.sharded.shape)
        else:
            self.flat_grad.add_(red)


def _register_post_backward(state: _FSDPState) -> None:
    """Run the unit's gradient reduction once all of the gathered tensors of this forward have
    received their gradient (the role of RegisterPostBackwardFunction,
    tensorplay/distributed/fsdp/_fully_shard/_fsdp_param_group.py:989-1006)."""
    fulls = [p.unsharded for p in state.params]
    live = [t for t in fulls if t is not None and t.requires_grad]
    pending = {"n": len(live)}
    total = len(live)

    def hook(_):
        pending["n"] -= 1
        if pending["n"] == 0:
            pending["n"] = total
            state.post_backward(fulls)

    for t in live:
        # a unit kept gathered across forwards reuses its tensors: one set of hooks serves them all
        if not getattr(t, "_tpb_hooked", False):
            t.register_post_accumulate_grad_hook(hook)
            t._tpb_hooked = True


# ------------------------------------------------------------------------------------------ module mixin
class FSDPModule:
    """Mixin added to a sharded module's class (the class is swapped in place, as in the
    reference: ``<Cls>FSDPModule(FSDPModule, Cls)``)."""

    def _states(self, recurse: bool) -> Iterable[_FSDPState]:
        return self._fsdp_state.tree(recurse)

    def unshard(self, async_op: bool = False):
        self._fsdp_state.unshard()
        return UnshardHandle() if async_op else None

    def reshard(self) -> None:
        self._fsdp_state.reshard()

    def reset_iter_state(self) -> None:
        for st in self._states(True):
            st.unreduced = st.partial = None

    def set_requires_gradient_sync(self, requires: bool, *, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.reduce_grads = requires

    def set_requires_all_reduce(self, requires: bool, *, recurse: bool = True) -> None:
        """Hybrid sharding only: with ``False`` the reduce-scattered gradients are accumulated and the
        all-reduce over the replicas waits until it is switched on again."""
        for st in self._states(recurse):
            st.requires_all_reduce = requires

    def set_is_last_backward(self, is_last: bool) -> None:
        self._fsdp_state.is_last_backward = is_last

    def set_reshard_after_forward(self, reshard: bool, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.reshard_after_forward = bool(reshard)

    def set_reshard_after_backward(self, reshard: bool, *, recurse: bool = True) -> None:
        for st in self._states(recurse):
            st.reshard_after_backward = reshard

    def set_gradient_divide_factor(self, factor: float) -> None:
        self._fsdp_state.divide = float(factor)

    def set_reduce_scatter_divide_factor(self, factor: float) -> None:
        self._fsdp_state.divide = float(factor)

    def set_force_sum_reduction_for_comms(self, enable: bool) -> None:
        self._fsdp_state.force_sum = bool(enable)

    def set_modules_to_forward_prefetch(self, modules) -> None:
        self._fsdp_state.fwd_prefetch = list(modules)

    def set_modules_to_backward_prefetch(self, modules) -> None:
        self._fsdp_state.bwd_prefetch = list(modules)

    def set_unshard_in_backward(self, unshard: bool) -> None:
        self._fsdp_state.unshard_in_backward = unshard

    def set_custom_all_gather(self, comm: AllGather) -> None:
        if not isinstance(comm, AllGather):
            raise TypeError("set_custom_all_gather expects an AllGather")
        self._fsdp_state.all_gather_comm = comm

    def set_custom_reduce_scatter(self, comm: ReduceScatter) -> None:
        if not isinstance(comm, ReduceScatter):
            raise TypeError("set_custom_reduce_scatter expects a ReduceScatter")
        self._fsdp_state.reduce_scatter_comm = comm

    def set_all_reduce_hook(self, hook: Callable[[torch.Tensor], None], *, stream=None) -> None:
        """``hook(reduced_shard)`` runs on the unit's reduced gradient (after the reduce-scatter, and
        after the all-reduce over replicas under hybrid sharding), before the division."""
        st = self._fsdp_state
        if stream is not None and st.replicate_group is not None:
            raise ValueError("a stream cannot be given together with hybrid sharding")
        st.all_reduce_hook, st.all_reduce_hook_stream = hook, stream

    def set_post_optim_event(self, event) -> None:
        self._fsdp_state.post_optim_event = event

    def set_allocate_memory_from_process_group_for_comm(self, enable: bool) -> None:
        if enable:
            raise NotImplementedError("process-group allocated communication buffers are not implemented; use "
                                      "set_custom_all_gather / set_custom_reduce_scatter with a Comm that allocates")

    def set_symm_mem_for_comm(self, backend: str = "NCCL") -> None:
        raise NotImplementedError("symmetric-memory transport of the public fully_shard is not wired; "
                                  "tensorplay_b200.parallel.FSDPEngine trains on the peer-memory kernels")

    def set_reduce_scatter_unused_params(self, enable: bool = True) -> None:
        pass  # parameters without a gradient already enter the reduction as zeros

    def _get_fsdp_state(self) -> _FSDPState:
        return self._fsdp_state


class UnshardHandle:
    """Returned by ``unshard(async_op=True)``; the gather here has completed when it returns."""

    def wait(self) -> None:
        return None


def register_fsdp_forward_method(module: nn.Module, method_name: str) -> None:
    """Make ``module.<method_name>(...)`` run the unit's pre- and post-forward logic like
    ``forward`` (tensorplay/distributed/fsdp/_fully_shard/_fully_shard.py:493-508)."""
    st = getattr(module, "_fsdp_state", None)
    if st is None:
        return
    orig = getattr(module, method_name)

    def wrapped(*args, **kwargs):
        args, kwargs = st.pre_forward(module, args, kwargs)
        return st.post_forward(module, args, orig(*args, **kwargs))

    object.__setattr__(module, method_name, wrapped)


def share_comm_ctx(modules: List[FSDPModule]) -> None:
    """Let several roots (pipeline stages of one rank) share one communication context."""
    if not modules:
        return
    for m in modules:
        if getattr(m, "_fsdp_state", None) is None:
            raise ValueError("share_comm_ctx expects modules that fully_shard was applied to")
    ctx = modules[0]._fsdp_state.comm_ctx
    for m in modules[1:]:
        for st in m._fsdp_state.tree(True):
            st.comm_ctx = ctx


# ------------------------------------------------------------------------------------------ fully_shard
def _groups_of(mesh, dp_mesh_dims: Optional[DataParallelMeshDims]):
    """(shard group, replicate group or None) of a 1-D or 2-D device mesh."""
    if mesh.ndim == 1:
        return mesh.get_group(), None
    if dp_mesh_dims is not None:
        names = mesh.mesh_dim_names
        def one(v):
            if v is None:
                return None
            v = v if isinstance(v, str) else (v[0] if len(v) == 1 else None)
            if v is None:
                raise NotImplementedError("several mesh dimensions per role are not implemented")
            return mesh.get_group(names.index(v))
        return one(dp_mesh_dims.shard), one(dp_mesh_dims.replicate)
    if mesh.ndim == 2:
        return mesh.get_group(1), mesh.get_group(0)  # (replicate, shard), the reference's HSDP convention
    raise ValueError("fully_shard expects a 1-D mesh, a 2-D (replicate, shard) mesh, or dp_mesh_dims naming the dims")


def fully_shard(module: Union[nn.Module, Sequence[nn.Module]], *, mesh=None,
                reshard_after_forward: Union[bool, int, None] = None, shard_placement_fn=None,
                mp_policy: Optional[MixedPrecisionPolicy] = None, offload_policy: Optional[OffloadPolicy] = None,
                ignored_params=None, dp_mesh_dims: Optional[DataParallelMeshDims] = None, process_group=None):
    """Shard ``module``'s parameters (those not already owned by an inner ``fully_shard`` unit)
    over the data-parallel group. Apply bottom-up: each block first, then the root.

    ``mesh``: 1-D (shard) or 2-D (replicate, shard: gradients are additionally all-reduced over the
    replicate dimension). ``reshard_after_forward``: ``None`` (root keeps its parameters, the other
    units free them), a bool, or - not implemented here - an int (resharding to a smaller group).
    """
    mods = [module] if isinstance(module, nn.Module) else list(module)
    if not mods:
        raise ValueError("fully_shard expects at least one module")
    root = mods[0]
    for m in mods:
        if getattr(m, "_fsdp_state", None) is not None:
            raise ValueError("fully_shard has already been applied to this module")
    if shard_placement_fn is not None:
        raise NotImplementedError("shard_placement_fn (sharding on another dimension than 0) is not implemented")
    if isinstance(reshard_after_forward, int) and not isinstance(reshard_after_forward, bool):
        raise NotImplementedError("an integer reshard_after_forward (resharding to a smaller group) is not implemented")
    mp_policy = mp_policy or MixedPrecisionPolicy()
    offload_policy = offload_policy or OffloadPolicy()
    group, rep_group = process_group, None
    if mesh is not None:
        group, rep_group = _groups_of(mesh, dp_mesh_dims)
    init = dist.is_available() and dist.is_initialized()
    world = dist.get_world_size(group) if init else 1
    rank = dist.get_rank(group) if init else 0
    ignored = {id(p) for p in (ignored_params or [])}
    infos: List[_ShardedParam] = []
    originals: List[nn.Parameter] = []
    seen = set()
    for m in mods:
        for sub in m.modules():
            if sub is not m and getattr(sub, "_fsdp_state", None) is not None:
                continue
            if _owned_by_inner(m, sub):
                continue
            for name, p in list(sub._parameters.items()):
                if p is None or id(p) in ignored or getattr(p, "_fsdp_info", None) is not None or id(p) in seen:
                    continue
                seen.add(id(p))
                infos.append(_ShardedParam(sub, name, p, world, rank))
                originals.append(p)
    has_inner = any(getattr(s, "_fsdp_state", None) is not None for m in mods for s in m.modules() if s is not m)
    if reshard_after_forward is None:
        reshard_after_forward = not has_inner  # the root's parameters are needed again at once in backward
    state = _FSDPState(root, infos, originals, group, rep_group, mp_policy, offload_policy, bool(reshard_after_forward))
    for m in mods:
        m._fsdp_state = state
        cls = m.__class__
        m.__class__ = type(cls.__name__ + "FSDPModule", (FSDPModule, cls), {})
    root.register_forward_pre_hook(state.pre_forward, with_kwargs=True, prepend=True)
    root.register_forward_hook(state.post_forward, prepend=False)
    return module


def _owned_by_inner(root: nn.Module, sub: nn.Module) -> bool:
    """True if ``sub`` sits below a descendant of ``root`` that is itself an FSDP unit."""
    for m in root.modules():
        if m is root:
            continue
        if getattr(m, "_fsdp_state", None) is not None:
            for d in m.modules():
                if d is sub:
                    return True
    return False


from .state_dict_api import StateDictMixin, StateDictSettings  # noqa: E402


# ------------------------------------------------------------------------------------------ FSDP1 facade
class FullyShardedDataParallel(StateDictMixin, nn.Module):
    """FSDP1-style wrapper implemented on ``fully_shard`` (the reference does the same,
    tensorplay/distributed/fsdp/fully_sharded_data_parallel.py:367-376). State-dict keys carry no
    extra prefix: ``full_state_dict`` returns full (unsharded) tensors on every rank."""

    def __init__(self, module: nn.Module, process_group=None, sharding_strategy=None, cpu_offload=None,
                 auto_wrap_policy=None, backward_prefetch=None, mixed_precision: Optional[MixedPrecision] = None,
                 ignored_modules=None, param_init_fn=None, device_id=None, sync_module_states: bool = False,
                 forward_prefetch: bool = False, limit_all_gathers: bool = True, use_orig_params: bool = True,
                 ignored_states=None, device_mesh=None):
        super().__init__()
        self._sd_settings = StateDictSettings()
        if not use_orig_params:
            raise NotImplementedError("use_orig_params=False (a FlatParameter per wrapper) is not implemented: the "
                                      "original parameters stay visible, sharded on dim 0")
        if sharding_strategy == ShardingStrategy.NO_SHARD:
            raise NotImplementedError("NO_SHARD is plain data parallelism: use DistributedDataParallel")
        if sharding_strategy in (ShardingStrategy.HYBRID_SHARD, ShardingStrategy._HYBRID_SHARD_ZERO2) and device_mesh is None:
            raise ValueError("hybrid sharding needs device_mesh=(replicate, shard)")
        self.module = module
        if param_init_fn is not None:
            for sub in module.modules():
                if any(p.is_meta for p in sub.parameters(recurse=False)):
                    param_init_fn(sub)
        if device_id is not None:
            dev = torch.device("cuda", device_id) if isinstance(device_id, int) else torch.device(device_id)
            module.to(dev)
        mp = MixedPrecisionPolicy(param_dtype=mixed_precision.param_dtype if mixed_precision else None,
                                  reduce_dtype=mixed_precision.reduce_dtype if mixed_precision else None)
        offload = CPUOffloadPolicy() if (cpu_offload is not None and cpu_offload.offload_params) else OffloadPolicy()
        ignored = []
        for im in (ignored_modules or []):
            ignored += list(im.parameters())
        ignored += [p for p in (ignored_states or []) if isinstance(p, nn.Parameter)]
        if sync_module_states and dist.is_initialized():
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t.data, src=dist.get_global_rank(process_group, 0) if process_group is not None else 0,
                               group=process_group)
        reshard = sharding_strategy not in (ShardingStrategy.SHARD_GRAD_OP, ShardingStrategy._HYBRID_SHARD_ZERO2)
        kw = dict(process_group=process_group if device_mesh is None else None, mp_policy=mp, mesh=device_mesh,
                  offload_policy=offload, ignored_params=ignored)
        wrapped = []
        if auto_wrap_policy is not None:
            for child in module.modules():
                if child is not module and auto_wrap_policy(child, False, sum(p.numel() for p in child.parameters())):
                    fully_shard(child, reshard_after_forward=reshard, **kw)
                    wrapped.append(child)
        fully_shard(module, reshard_after_forward=reshard if not wrapped else False, **kw)
        if forward_prefetch and wrapped:
            for a, b in zip(wrapped[:-1], wrapped[1:]):
                a.set_modules_to_forward_prefetch([b])
        self.backward_prefetch = backward_prefetch

    def forward(self, *a, **k):
        return self.module(*a, **k)

    @contextlib.contextmanager
    def no_sync(self):
        self.module.set_requires_gradient_sync(False)
        try:
            yield
        finally:
            self.module.set_requires_gradient_sync(True)

    @contextlib.contextmanager
    def summon_full_params(self, recurse: bool = True, writeback: bool = True):
        """Full parameters inside the block; with ``writeback`` in-place changes made to them are
        copied back into the local shards on exit (fully_sharded_data_parallel.py:783)."""
        states = [st for st in self.module._fsdp_state.tree(recurse)]
        for st in states:
            st.unshard()
        try:
            yield
        finally:
            for st in states:
                if writeback:
                    for p in st.params:
                        if p.unsharded is None or not p.local_rows:
                            continue
                        full2 = p.unsharded.detach().reshape(p.n0, p.rest_numel)
                        rows = full2[st.rank * p.chunk: st.rank * p.chunk + p.local_rows]
                        st.flat_shard[p.offset: p.offset + rows.numel()].copy_(rows.reshape(-1).to(st.flat_shard.dtype))
                st.reshard()

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        """Name -> full (unsharded) tensor of every parameter, on every rank."""
        out: Dict[str, torch.Tensor] = {}
        where = {}
        for name, mod in self.module.named_modules():
            where[id(mod)] = name
        with self.summon_full_params(writeback=False):
            for st in self.module._fsdp_state.tree(True):
                for p in st.params:
                    prefix = where.get(id(p.module), "")
                    out[(prefix + "." if prefix else "") + p.name] = p.unsharded.detach().clone()
        for name, b in self.module.named_buffers():
            out[name] = b.detach().clone()
        return out

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
        """Clip by the norm of the *global* gradient: the local shards' norms are combined over the
        shard group (fully_sharded_data_parallel.py:969)."""
        ps = [p for p in self.module.parameters() if p.grad is not None]
        dev = ps[0].grad.device if ps else torch.device("cpu")
        inf = norm_type == float("inf")
        if inf:
            local = torch.stack([p.grad.float().abs().max() for p in ps]).max() if ps else torch.zeros((), device=dev)
        else:
            local = torch.stack([p.grad.float().norm(norm_type) ** norm_type for p in ps]).sum() if ps else torch.zeros((), device=dev)
        st = self.module._fsdp_state
        if dist.is_initialized() and st.world > 1:
            red = local.to(st.device) if st.cpu_offload else local
            dist.all_reduce(red, op=dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM, group=st.group)
            local = red.to(dev)
        total = local if inf else local ** (1.0 / norm_type)
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        for p in ps:
            p.grad.mul_(coef.to(p.grad.dtype))
        return total
