from __future__ import annotations

import contextlib
import enum
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Union

import torch
import torch.distributed as dist
from torch import nn


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
    pin_memory: bool = True


class ShardingStrategy(enum.Enum):
    FULL_SHARD = 1
    SHARD_GRAD_OP = 2
    NO_SHARD = 3
    HYBRID_SHARD = 4


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


def _chunk_sizes(n0: int, world: int):
    """Ceil-chunking of dim 0 with empty tail chunks (torch.chunk semantics)."""
    c = (n0 + world - 1) // world
    return c, [max(0, min(c, n0 - r * c)) for r in range(world)]


class _ShardedParam:
    """Book-keeping for one parameter: its padded local shard and how to rebuild the full tensor."""

    def __init__(self, module: nn.Module, name: str, param: nn.Parameter, group, world: int, rank: int,
                 mp: MixedPrecisionPolicy):
        self.module, self.name = module, name
        self.full_shape = tuple(param.shape)
        self.orig_dtype = param.dtype
        self.group, self.world, self.rank = group, world, rank
        self.mp = mp
        n0 = self.full_shape[0] if len(self.full_shape) else 1
        data = param.data if param.dim() else param.data.reshape(1)
        self.chunk, sizes = _chunk_sizes(n0, world)
        self.local_rows = sizes[rank]
        rest = tuple(data.shape[1:])
        padded = torch.zeros((self.chunk,) + rest, dtype=param.dtype, device=param.device)
        if self.local_rows:
            padded[: self.local_rows].copy_(data[rank * self.chunk: rank * self.chunk + self.local_rows])
        self.padded = padded
        # the sharded parameter keeps its identity across unshard / reshard (optimizers hold it)
        self.sharded = nn.Parameter(padded[: self.local_rows], requires_grad=param.requires_grad)
        self.sharded._fsdp_info = self
        self.unsharded: Optional[torch.Tensor] = None
        setattr_param(module, name, self.sharded)

    def all_gather(self) -> None:
        src = self.padded
        dt = self.mp.param_dtype or self.orig_dtype
        if src.dtype != dt:
            src = src.to(dt)
        out = torch.empty((self.world * self.chunk,) + tuple(src.shape[1:]), dtype=dt, device=src.device)
        if self.world > 1:
            dist.all_gather_into_tensor(out, src.contiguous(), group=self.group)
        else:
            out.copy_(src)
        n0 = self.full_shape[0] if len(self.full_shape) else 1
        full = out[:n0].reshape(self.full_shape)
        self.unsharded = full.requires_grad_(self.sharded.requires_grad)
        # plain tensor attribute (not a registered parameter) for the duration of the compute
        self.module._parameters.pop(self.name, None)
        object.__setattr__(self.module, self.name, self.unsharded)

    def reshard(self) -> None:
        if self.name in self.module.__dict__:
            del self.module.__dict__[self.name]
        self.module._parameters[self.name] = self.sharded
        self.unsharded = None

    def reduce_scatter_grad(self, divide: float, reduce_grads: bool = True, full: Optional[torch.Tensor] = None) -> None:
        """Reduce the gradient held by ``full`` (the gathered tensor one forward computed with; the
        currently gathered one by default) into the shard's ``.grad``, accumulating."""
        full = full if full is not None else self.unsharded
        g = full.grad if full is not None else None
        if g is None:
            return
        full.grad = None
        acc = getattr(self, "unreduced", None)
        if not reduce_grads:
            # gradient synchronisation is off (accumulation steps): keep the full-size sum locally
            # until a backward with synchronisation on reduces it
            self.unreduced = g if acc is None else acc.add_(g)
            return
        if acc is not None:
            g = acc.add_(g)
            self.unreduced = None
        rd = self.mp.reduce_dtype or g.dtype
        n0 = self.full_shape[0] if len(self.full_shape) else 1
        g2 = g.reshape((n0,) + tuple(g.shape[1:]) if g.dim() else (1,)).to(rd)
        if self.world * self.chunk == n0:
            padded = g2.contiguous()
        else:
            padded = torch.zeros((self.world * self.chunk,) + tuple(g2.shape[1:]), dtype=rd, device=g.device)
            padded[:n0].copy_(g2)
        if self.world > 1:
            out = torch.empty((self.chunk,) + tuple(g2.shape[1:]), dtype=rd, device=g.device)
            if dist.get_backend(self.group) == "gloo":
                dist.all_reduce(padded, group=self.group)
                out.copy_(padded[self.rank * self.chunk: (self.rank + 1) * self.chunk])
            else:
                dist.reduce_scatter_tensor(out, padded, group=self.group)
            out.div_(divide)
        else:
            out = padded[self.rank * self.chunk: (self.rank + 1) * self.chunk]
        shard_grad = out[: self.local_rows].to(self.orig_dtype)
        if self.sharded.grad is None:
            self.sharded.grad = shard_grad.reshape(self.sharded.shape).clone()
        else:
            self.sharded.grad.add_(shard_grad.reshape(self.sharded.shape))


def setattr_param(module: nn.Module, name: str, p: nn.Parameter) -> None:
    module._parameters[name] = p


class FSDPModule:
    """Mixin added to a sharded module's class (the class is swapped in place, as in the
    reference: ``<Cls>FSDPModule(FSDPModule, Cls)``)."""

    def unshard(self, async_op: bool = False):
        self._fsdp_state.unshard()
        return None

    def reshard(self) -> None:
        self._fsdp_state.reshard()

    def set_requires_gradient_sync(self, requires: bool, *, recurse: bool = True) -> None:
        for st in self._fsdp_state.tree(recurse):
            st.reduce_grads = requires

    def set_is_last_backward(self, is_last: bool) -> None:
        self._fsdp_state.is_last_backward = is_last

    def set_reshard_after_forward(self, reshard: bool, recurse: bool = True) -> None:
        for st in self._fsdp_state.tree(recurse):
            st.reshard_after_forward = reshard

    def set_reshard_after_backward(self, reshard: bool, *, recurse: bool = True) -> None:
        for st in self._fsdp_state.tree(recurse):
            st.reshard_after_backward = reshard

    def set_gradient_divide_factor(self, factor: float) -> None:
        self._fsdp_state.divide = float(factor)

    def set_modules_to_forward_prefetch(self, modules) -> None:
        self._fsdp_state.fwd_prefetch = list(modules)

    def set_modules_to_backward_prefetch(self, modules) -> None:
        self._fsdp_state.bwd_prefetch = list(modules)

    def set_requires_all_reduce(self, requires: bool, *, recurse: bool = True) -> None:
        pass  # only meaningful for hybrid sharding (replicate dimension)

    def set_unshard_in_backward(self, unshard: bool) -> None:
        self._fsdp_state.unshard_in_backward = unshard


class _FSDPState:
    def __init__(self, module: nn.Module, params: List[_ShardedParam], world: int, reshard_after_forward: bool):
        self.module, self.params, self.world = module, params, world
        self.reshard_after_forward = reshard_after_forward
        self.reshard_after_backward = True
        self.reduce_grads = True
        self.is_last_backward = True
        self.unshard_in_backward = True
        self.divide = float(world)
        self.is_unsharded = False
        self.fwd_prefetch: list = []
        self.bwd_prefetch: list = []
        self.children: List["_FSDPState"] = []

    def tree(self, recurse: bool):
        yield self
        if recurse:
            for m in self.module.modules():
                st = getattr(m, "_fsdp_state", None)
                if st is not None and st is not self:
                    yield st

    def unshard(self) -> None:
        if not self.is_unsharded:
            for p in self.params:
                p.all_gather()
            self.is_unsharded = True

    def reshard(self) -> None:
        if self.is_unsharded:
            for p in self.params:
                p.reshard()
            self.is_unsharded = False

    # hooks
    def pre_forward(self, module, args, kwargs):
        self.unshard()
        for m in self.fwd_prefetch:
            m._fsdp_state.unshard()
        if torch.is_grad_enabled():
            tensors = [a for a in args if isinstance(a, torch.Tensor) and a.requires_grad]
            self._saved_unsharded = [p.unsharded for p in self.params]
        return args, kwargs

    def post_forward(self, module, args, output):
        need_bwd = torch.is_grad_enabled() and any(p.sharded.requires_grad for p in self.params)
        if need_bwd:
            output = _register_post_backward(self, output)
        if self.reshard_after_forward and not need_bwd:
            self.reshard()
        elif self.reshard_after_forward and need_bwd:
            # keep the autograd graph's references to the gathered tensors; they are re-bound in
            # backward, and the module goes back to its sharded parameters now
            for p in self.params:
                p.kept = p.unsharded
                p.reshard()
            self.is_unsharded = False
        return output

    def post_backward(self, fulls: Optional[list] = None) -> None:
        """``fulls``: the gathered tensors of the forward whose backward just finished. Several
        forwards may precede the first backward (pipeline micro-batches), each with its own gathered
        copies, so the gradients are read from the copies that forward used."""
        for i, p in enumerate(self.params):
            full = fulls[i] if fulls is not None else (
                p.unsharded if p.unsharded is not None else getattr(p, "kept", None))
            if full is None:
                continue
            p.reduce_scatter_grad(self.divide, self.reduce_grads, full)
            if getattr(p, "kept", None) is full:
                p.kept = None
        if self.reshard_after_backward:
            self.reshard()


class _PostBackward(torch.autograd.Function):
    """Identity on the unit's inputs whose backward fires after the unit's parameter gradients
    are complete (the role of RegisterPostBackwardFunction,
    tensorplay/distributed/fsdp/_fully_shard/_fsdp_param_group.py:989-1006)."""

    @staticmethod
    def forward(ctx, state, *inputs):
        ctx.state = state
        return inputs

    @staticmethod
    def backward(ctx, *grads):
        ctx.state.post_backward()
        return (None,) + grads


def _register_post_backward(state: _FSDPState, output):
    # Hook a callback on the module's parameters' accumulation: run post_backward once all of the
    # unit's unsharded tensors have received their gradient.
    fulls = [p.unsharded for p in state.params]
    pending = {"n": sum(1 for t in fulls if t is not None and t.requires_grad)}
    total = pending["n"]

    def hook(_):
        pending["n"] -= 1
        if pending["n"] == 0:
            pending["n"] = total
            state.post_backward(fulls)

    for t in fulls:
        # a unit kept gathered across forwards reuses its tensors: one set of hooks serves them all
        if t is not None and t.requires_grad and not getattr(t, "_tpb_hooked", False):
            t.register_post_accumulate_grad_hook(hook)
            t._tpb_hooked = True
    return output


def fully_shard(module: Union[nn.Module, Sequence[nn.Module]], *, mesh=None, reshard_after_forward: bool = True,
                mp_policy: MixedPrecisionPolicy = MixedPrecisionPolicy(), offload_policy: OffloadPolicy = OffloadPolicy(),
                shard_placement_fn=None, ignored_params=None, process_group=None):
    """Shard ``module``'s parameters (those not already owned by an inner ``fully_shard`` unit)
    over the data-parallel group. Apply bottom-up: each block first, then the root."""
    mods = [module] if isinstance(module, nn.Module) else list(module)
    root = mods[0]
    if getattr(root, "_fsdp_state", None) is not None:
        raise ValueError("fully_shard has already been applied to this module")
    group = process_group
    if mesh is not None:
        group = mesh.get_group() if mesh.ndim == 1 else mesh.get_group(mesh.ndim - 1)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    ignored = {id(p) for p in (ignored_params or [])}
    params: List[_ShardedParam] = []
    for m in mods:
        for sub in m.modules():
            if sub is not m and getattr(sub, "_fsdp_state", None) is not None:
                continue
            for name, p in list(sub._parameters.items()):
                if p is None or id(p) in ignored or getattr(p, "_fsdp_info", None) is not None:
                    continue
                if _owned_by_inner(m, sub):
                    continue
                params.append(_ShardedParam(sub, name, p, group, world, rank, mp_policy))
    state = _FSDPState(root, params, world, bool(reshard_after_forward))
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


class FullyShardedDataParallel(nn.Module):
    """FSDP1-style wrapper implemented on ``fully_shard`` (the reference does the same,
    tensorplay/distributed/fsdp/fully_sharded_data_parallel.py:367-376). State-dict keys carry no
    extra prefix: ``state_dict`` returns full (unsharded) tensors on every rank."""

    def __init__(self, module: nn.Module, process_group=None, sharding_strategy=None, cpu_offload=None,
                 auto_wrap_policy=None, backward_prefetch=None, mixed_precision: Optional[MixedPrecision] = None,
                 ignored_modules=None, param_init_fn=None, device_id=None, sync_module_states: bool = False,
                 forward_prefetch: bool = False, limit_all_gathers: bool = True, use_orig_params: bool = True,
                 ignored_states=None, device_mesh=None):
        super().__init__()
        self.module = module
        mp = MixedPrecisionPolicy(param_dtype=mixed_precision.param_dtype if mixed_precision else None,
                                  reduce_dtype=mixed_precision.reduce_dtype if mixed_precision else None)
        if sync_module_states and dist.is_initialized():
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t.data, src=0, group=process_group)
        if auto_wrap_policy is not None:
            for child in module.modules():
                if child is not module and auto_wrap_policy(child, False, sum(p.numel() for p in child.parameters())):
                    fully_shard(child, process_group=process_group, mp_policy=mp, mesh=device_mesh)
        reshard = sharding_strategy not in (ShardingStrategy.SHARD_GRAD_OP, ShardingStrategy.NO_SHARD)
        fully_shard(module, process_group=process_group, mp_policy=mp, mesh=device_mesh,
                    reshard_after_forward=reshard)

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
    def summon_full_params(self, recurse: bool = True, writeback: bool = False):
        states = list(self.module._fsdp_state.tree(recurse))
        for st in states:
            st.unshard()
        try:
            yield
        finally:
            for st in states:
                st.reshard()

    def full_state_dict(self) -> Dict[str, torch.Tensor]:
        with self.summon_full_params():
            out = {}
            for st in self.module._fsdp_state.tree(True):
                for p in st.params:
                    pass
            for name, mod in self.module.named_modules():
                for pname, t in list(mod.__dict__.items()):
                    if isinstance(t, torch.Tensor) and any(sp.module is mod and sp.name == pname for st in self.module._fsdp_state.tree(True) for sp in st.params):
                        out[(name + "." if name else "") + pname] = t.detach().clone()
            return out

    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
        ps = [p for p in self.module.parameters() if p.grad is not None]
        local = torch.stack([p.grad.float().norm(norm_type) ** norm_type for p in ps]).sum() if ps else torch.zeros(())
        if dist.is_initialized():
            dist.all_reduce(local)
        total = local ** (1.0 / norm_type)
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        for p in ps:
            p.grad.mul_(coef.to(p.grad.dtype))
        return total
