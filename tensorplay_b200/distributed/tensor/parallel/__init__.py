"""Tensor / sequence parallel styles and ``parallelize_module``.

``ColwiseParallel`` / ``RowwiseParallel`` shard ``nn.Linear`` weights across the TP group and
replace the module's forward with the fused kernels of ``tensorplay_b200.parallel.tp``
(all-gather->GEMM for column-parallel layers fed by sequence-sharded activations,
GEMM->reduce-scatter for row-parallel layers); on CPU ranks the same styles run plain collectives.
``SequenceParallel`` marks norm-like modules as operating on sequence shards (their parameters
stay replicated and their gradients are all-reduced). Names follow
tensorplay/distributed/tensor/parallel/api.py:16-55 and style.py:67-218.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Optional, Union

import torch
import torch.distributed as dist
from torch import nn

from ....parallel.tp import TPContext, _AllGatherRows, _ReduceScatterRows

__all__ = ["ParallelStyle", "ColwiseParallel", "RowwiseParallel", "SequenceParallel", "PrepareModuleInput",
           "PrepareModuleOutput", "PrepareModuleInputOutput", "input_reshard", "parallelize_module", "loss_parallel"]


class ParallelStyle:
    def apply(self, module: nn.Module, ctx: TPContext) -> nn.Module:
        raise NotImplementedError


def _shard_rows(w: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    assert w.shape[0] % world == 0, "dimension not divisible by the TP degree"
    n = w.shape[0] // world
    return w[rank * n: (rank + 1) * n].clone()


class ColwiseParallel(ParallelStyle):
    """Weight ``[out, in]`` sharded on ``out``. ``input_sharded=True``: the input arrives
    sequence-sharded ``[rows/world, in]`` and is all-gathered inside the GEMM kernel; otherwise the
    input is replicated and the layer is a local GEMM. Output: ``[rows, out/world]``."""

    def __init__(self, *, input_sharded: bool = True):
        self.input_sharded = input_sharded

    def apply(self, module: nn.Linear, ctx: TPContext) -> nn.Module:
        w, r = ctx.world, ctx.rank
        module.weight = nn.Parameter(_shard_rows(module.weight.data, w, r))
        if module.bias is not None:
            module.bias = nn.Parameter(_shard_rows(module.bias.data, w, r))
        sharded = self.input_sharded

        def forward(x):
            shape = x.shape
            x2 = x.reshape(-1, shape[-1])
            if sharded and w > 1:
                y = ctx.all_gather_linear(x2, module.weight)
            else:
                if w > 1:
                    # replicated input: every rank back-propagates only its columns' share of dx
                    x2 = _CopyToRegion.apply(x2, ctx.group)
                y = torch.nn.functional.linear(x2, module.weight) if not x2.is_cuda else _local_linear(x2, module.weight)
            if module.bias is not None:
                y = y + module.bias
            # a replicated input keeps its leading dimensions; sequence shards stay [rows, out / world]
            return y if (sharded and w > 1) else y.view(*shape[:-1], y.shape[-1])
        module.forward = forward
        module._tp_style = "colwise"
        return module


class RowwiseParallel(ParallelStyle):
    """Weight ``[out, in]`` sharded on ``in``; the input is ``[rows, in/world]``. With
    ``output_sharded=True`` the partial products are reduce-scattered over rows inside the GEMM
    kernel (sequence parallel output ``[rows/world, out]``), otherwise all-reduced."""

    def __init__(self, *, output_sharded: bool = True):
        self.output_sharded = output_sharded

    def apply(self, module: nn.Linear, ctx: TPContext) -> nn.Module:
        w, r = ctx.world, ctx.rank
        module.weight = nn.Parameter(_shard_rows(module.weight.data.t().contiguous(), w, r).t().contiguous())
        scattered = self.output_sharded

        def forward(x):
            shape = x.shape
            x2 = x.reshape(-1, shape[-1])
            if w == 1:
                y = torch.nn.functional.linear(x2, module.weight)
            elif scattered:
                y = ctx.linear_reduce_scatter(x2, module.weight)
            else:
                y = _AllReduce.apply(torch.nn.functional.linear(x2, module.weight), ctx.group)
            if module.bias is not None:
                y = y + module.bias
            return y if (scattered and w > 1) else y.view(*shape[:-1], y.shape[-1])
        module.forward = forward
        module._tp_style = "rowwise"
        return module


class SequenceParallel(ParallelStyle):
    """Norm / dropout style: runs unchanged on the local sequence shard; parameter gradients are
    summed over the TP group after backward (``sync_grads``)."""

    def apply(self, module: nn.Module, ctx: TPContext) -> nn.Module:
        for p in module.parameters():
            p._tp_replicated = True
        return module


class _GatherToReplicate(torch.autograd.Function):
    """Row shards -> replicated tensor. The gradient of a replicated tensor is the same on every
    rank, so backward keeps this rank's rows (no reduction)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = x.new_empty(x.shape[0] * w, *x.shape[1:])
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = g.shape[0] // w
        return g[r * n: (r + 1) * n].contiguous(), None


class _SliceToShard(torch.autograd.Function):
    """Replicated tensor -> this rank's rows; backward gathers the row gradients of all ranks."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w, r = dist.get_world_size(group), dist.get_rank(group)
        assert x.shape[0] % w == 0, "rows not divisible by the tensor-parallel degree"
        n = x.shape[0] // w
        return x[r * n: (r + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = g.new_empty(g.shape[0] * w, *g.shape[1:])
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def _layout_name(layout) -> str:
    """``"shard"`` / ``"replicate"`` from a string or a placement object (``Shard(0)``, ``Replicate()``)."""
    name = layout if isinstance(layout, str) else type(layout).__name__
    name = name.lower()
    if name.startswith("shard"):
        return "shard"
    if name.startswith("replicate"):
        return "replicate"
    raise ValueError(f"unknown layout {layout!r}")


def _convert(t, src, dst, ctx: TPContext):
    if not isinstance(t, torch.Tensor) or src is None or dst is None or ctx.world == 1:
        return t
    a, b = _layout_name(src), _layout_name(dst)
    if a == b:
        return t
    return _GatherToReplicate.apply(t, ctx.group) if a == "shard" else _SliceToShard.apply(t, ctx.group)


def _as_tuple(x, n):
    if isinstance(x, (tuple, list)):
        return tuple(x)
    return (x,) * n if n else (x,)


class PrepareModuleInput(ParallelStyle):
    """Convert the layouts of a module's positional inputs before its forward: ``"shard"`` (rows of
    dimension 0 split over the group) or ``"replicate"``; ``None`` leaves an argument alone."""

    def __init__(self, *, input_layouts=None, desired_input_layouts=None):
        self.src, self.dst = input_layouts, desired_input_layouts

    def apply(self, module: nn.Module, ctx: TPContext) -> nn.Module:
        def pre(mod, args):
            src, dst = _as_tuple(self.src, len(args)), _as_tuple(self.dst, len(args))
            return tuple(_convert(a, src[i] if i < len(src) else None, dst[i] if i < len(dst) else None, ctx)
                         for i, a in enumerate(args))
        module.register_forward_pre_hook(pre)
        return module


class PrepareModuleOutput(ParallelStyle):
    """Convert the layouts of a module's outputs after its forward."""

    def __init__(self, *, output_layouts=None, desired_output_layouts=None):
        self.src, self.dst = output_layouts, desired_output_layouts

    def apply(self, module: nn.Module, ctx: TPContext) -> nn.Module:
        def post(mod, args, out):
            if isinstance(out, tuple):
                src, dst = _as_tuple(self.src, len(out)), _as_tuple(self.dst, len(out))
                return tuple(_convert(o, src[i] if i < len(src) else None, dst[i] if i < len(dst) else None, ctx)
                             for i, o in enumerate(out))
            return _convert(out, _as_tuple(self.src, 1)[0], _as_tuple(self.dst, 1)[0], ctx)
        module.register_forward_hook(post)
        return module


class PrepareModuleInputOutput(ParallelStyle):
    def __init__(self, *, input_layouts=None, desired_input_layouts=None, output_layouts=None,
                 desired_output_layouts=None):
        self.inp = PrepareModuleInput(input_layouts=input_layouts, desired_input_layouts=desired_input_layouts)
        self.out = PrepareModuleOutput(output_layouts=output_layouts, desired_output_layouts=desired_output_layouts)

    def apply(self, module: nn.Module, ctx: TPContext) -> nn.Module:
        return self.out.apply(self.inp.apply(module, ctx), ctx)


def input_reshard(module: nn.Module, tp_device_mesh=None, input_reshard_dim: Optional[int] = 0, *, group=None) -> nn.Module:
    """Keep only this rank's slice (along ``input_reshard_dim``) of the replicated input that a
    tensor-parallel module saves for backward, and all-gather it when backward needs it: activation
    memory of the saved inputs drops by the tensor-parallel degree."""
    if input_reshard_dim is None:
        return module
    if tp_device_mesh is not None:
        group = tp_device_mesh.get_group()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return module
    rank = dist.get_rank(group)
    state = {}

    def pre(mod, args):
        first = args[0] if args and isinstance(args[0], torch.Tensor) else None
        marker = first.data_ptr() if first is not None else None
        shape = tuple(first.shape) if first is not None else None

        def pack(t):
            if (marker is not None and t.data_ptr() == marker and tuple(t.shape) == shape
                    and t.shape[input_reshard_dim] % world == 0):
                n = t.shape[input_reshard_dim] // world
                return ("shard", t.narrow(input_reshard_dim, rank * n, n).clone())
            return ("full", t)

        def unpack(item):
            kind, t = item
            if kind == "full":
                return t
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous(), group=group)
            return torch.cat(parts, dim=input_reshard_dim)
        cm = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
        cm.__enter__()
        state["cm"] = cm

    def post(mod, args, out):
        cm = state.pop("cm", None)
        if cm is not None:
            cm.__exit__(None, None, None)
    module.register_forward_pre_hook(pre)
    module.register_forward_hook(post)
    return module


def _local_linear(x, w):
    from .... import ops
    return ops.linear(x, w)


class _CopyToRegion(torch.autograd.Function):
    """Identity in forward, all-reduce of the gradient in backward (entry of a tensor-parallel region
    whose input is replicated)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


def parallelize_module(module: nn.Module, device_mesh=None, parallelize_plan: Union[ParallelStyle, Dict[str, ParallelStyle], None] = None,
                       *, tp_context: Optional[TPContext] = None) -> nn.Module:
    """Apply styles to sub-modules selected by fnmatch-style dotted paths."""
    group = None
    if device_mesh is not None:
        group = device_mesh.get_group() if device_mesh.ndim == 1 else device_mesh.get_group(device_mesh.ndim - 1)
    ctx = tp_context or TPContext(group=group)
    module._tp_context = ctx
    if parallelize_plan is None:
        return module
    if isinstance(parallelize_plan, ParallelStyle):
        return parallelize_plan.apply(module, ctx)
    names = dict(module.named_modules())
    for pattern, style in parallelize_plan.items():
        matched = [n for n in names if fnmatch.fnmatch(n, pattern)]
        if not matched:
            raise ValueError(f"parallelize_plan key {pattern!r} matches no sub-module")
        for n in matched:
            style.apply(names[n], ctx)
    # attention modules whose projections were sharded over heads now own num_heads / world heads
    for m in module.modules():
        q = getattr(m, "q_proj", None)
        if (q is not None and getattr(q, "_tp_style", None) == "colwise" and hasattr(m, "num_heads")
                and not getattr(m, "_tp_heads_local", False)):
            if m.num_heads % ctx.world or getattr(m, "num_kv_heads", ctx.world) % ctx.world:
                raise ValueError("the head counts must be divisible by the tensor-parallel degree")
            m.num_heads //= ctx.world
            if hasattr(m, "num_kv_heads"):
                m.num_kv_heads //= ctx.world
            m._tp_heads_local = True
    return module


def sync_replicated_grads(module: nn.Module) -> None:
    """Sum the gradients of parameters that are replicated across the TP group but saw only a
    sequence shard of the activations (``SequenceParallel`` modules)."""
    ctx = getattr(module, "_tp_context", None)
    if ctx is None or ctx.world == 1:
        return
    for p in module.parameters():
        if getattr(p, "_tp_replicated", False) and p.grad is not None:
            dist.all_reduce(p.grad, group=ctx.group)


class loss_parallel:
    """Context manager: cross-entropy over vocabulary-sharded logits ``[rows, V/world]``
    (column-parallel LM head) without gathering them: max and sum-exp are all-reduced."""

    def __init__(self, group=None):
        self.group = group

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False

    def cross_entropy(self, logits_shard: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        return _VocabParallelCE.apply(logits_shard, target, self.group)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, group):
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        lf = logits.float()
        vs = lf.shape[-1]
        m = lf.max(dim=-1).values
        if world > 1:
            dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
        e = torch.exp(lf - m[:, None])
        s = e.sum(-1)
        lo = rank * vs
        mine = (target >= lo) & (target < lo + vs)
        tl = torch.zeros_like(m)
        idx = (target - lo).clamp(0, vs - 1)
        tl[mine] = lf.gather(1, idx[:, None]).squeeze(1)[mine]
        if world > 1:
            dist.all_reduce(s, group=group)
            dist.all_reduce(tl, group=group)
        lse = m + s.log()
        ctx.save_for_backward(e / s[:, None], mine, idx)
        return (lse - tl).mean()

    @staticmethod
    def backward(ctx, g):
        p, mine, idx = ctx.saved_tensors
        grad = p.clone()
        rows = torch.arange(p.shape[0], device=p.device)[mine]
        grad[rows, idx[mine]] -= 1.0
        return (grad * (g / p.shape[0])).to(p.dtype), None, None
