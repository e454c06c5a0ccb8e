"""Flat-buffer fully-sharded training engine (ZeRO-3 style) with the optimizer fused into backward.

Design (one process per GPU):

* The model is cut into *units* (embedding, each transformer block, head). Every unit owns one
  flat bf16 parameter buffer; the module's parameters are views into it, so a unit is
  all-gathered as a single contiguous range and its GEMMs read the gathered buffer directly -
  there is no copy-in / copy-out as in the reference's ``foreach_all_gather`` +
  ``foreach_all_gather_copy_out`` (tensorplay/distributed/fsdp/_fully_shard/_fsdp_collectives.py:337-470).
* Each rank keeps only its 1/N shard of the fp32 master weights and Adam moments.
* Backward of a unit writes weight gradients straight into a flat bf16 gradient buffer (the
  GEMM / norm kernels take the destination view), then ONE fused step reduces the unit's
  gradients across ranks, scales, applies AdamW on the owned shard and emits the new bf16
  parameters - the reference runs cast + chunk_cat + ncclReduceScatter + divide + views
  (:473-690) and later a separate multi-tensor AdamW (p10/include/OptimizerMTA.cuh:627).
* Activation checkpointing per unit: forward keeps only the unit input; backward re-gathers
  the parameters (prefetching the next unit on the communication stream) and recomputes.

Communication backends: ``single`` (one rank), ``torch`` (torch.distributed all-gather /
reduce-scatter, gloo or NCCL: the baseline and the CPU test path) and ``symm`` (the fused
peer-memory kernels of ``tensorplay_b200.parallel.symm``).
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import Tensor, nn

from .. import ops
from ..ops import _ckpt


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


@dataclass
class AdamWConfig:
    lr: float = 3e-4
    betas: Tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.1


class ParamUnit:
    """One shardable group of parameters living in a flat buffer."""

    def __init__(self, index: int, name: str, params: List[Tuple[str, nn.Parameter]], world: int,
                 rank: int, device, param_dtype: torch.dtype):
        self.index, self.name, self.params = index, name, params
        self.world, self.rank = world, rank
        self.offsets: List[int] = []
        self.shapes = [tuple(p.shape) for _, p in params]
        self.numels = [p.numel() for _, p in params]
        off = 0
        for n in self.numels:
            self.offsets.append(off)
            off += _round_up(n, 8)  # keep every view 16-byte aligned
        self.numel = off
        self.padded = _round_up(max(off, 8), world * 128)
        self.shard_numel = self.padded // world
        self.device, self.param_dtype = device, param_dtype
        # state filled in by the engine
        self.full: Optional[Tensor] = None
        self.grad: Optional[Tensor] = None
        self.shard: Optional[Tensor] = None
        self.master: Optional[Tensor] = None
        self.exp_avg: Optional[Tensor] = None
        self.exp_avg_sq: Optional[Tensor] = None
        self.gather_event = None
        self.update_event = None
        self.local: Optional["ParamUnit"] = None
        self.red: Optional[Tensor] = None  # reduced gradient shard kept for a clipped (two-phase) step

    def bind_params(self, full: Tensor) -> None:
        self.full = full
        for (_, p), off, n, shape in zip(self.params, self.offsets, self.numels, self.shapes):
            p.data = full[off: off + n].view(shape)

    def bind_grads(self, grad: Optional[Tensor]) -> None:
        self.grad = grad
        for (_, p), off, n, shape in zip(self.params, self.offsets, self.numels, self.shapes):
            p._tpb_grad_view = None if grad is None else grad[off: off + n].view(shape)
            p._tpb_grad_written = False

    def collect_autograd_grads(self) -> None:
        """Fold ``.grad`` tensors produced by plain autograd paths into the flat buffer and zero the
        views that nothing wrote (the buffer itself is not cleared before backward: the kernels'
        first write to a view overwrites it)."""
        for _, p in self.params:
            v = p._tpb_grad_view
            if p.grad is not None:
                if getattr(p, "_tpb_grad_written", False):
                    v.add_(p.grad.to(v.dtype))
                else:
                    v.copy_(p.grad)
                    p._tpb_grad_written = True
                p.grad = None
            elif v is not None and not getattr(p, "_tpb_grad_written", False):
                v.zero_()

    def zero_padding(self, grad: Tensor) -> None:
        """Clear the alignment gaps and the tail of a freshly bound gradient buffer."""
        end = 0
        for off, n in zip(self.offsets, self.numels):
            if off > end:
                grad[end:off].zero_()
            end = off + n
        if end < grad.numel():
            grad[end:].zero_()

    def shard_range(self, rank: Optional[int] = None) -> Tuple[int, int]:
        r = self.rank if rank is None else rank
        return r * self.shard_numel, (r + 1) * self.shard_numel


class _UnitFn(torch.autograd.Function):
    """Runs one unit; with checkpointing only the inputs are kept and forward is recomputed."""

    @staticmethod
    def forward(ctx, engine, unit_idx, fn, checkpoint, n_tensor, *args):
        tensors, extra = args[:n_tensor], args[n_tensor:]
        ctx.engine, ctx.unit_idx, ctx.fn, ctx.checkpoint, ctx.extra = engine, unit_idx, fn, checkpoint, extra
        engine._pre_forward(unit_idx)
        ctx.kept = None
        if checkpoint == "selective":
            # GEMM and attention outputs are kept, the cheap ops in between are recomputed
            with torch.no_grad(), _ckpt.record() as kept:
                out = fn(*tensors, *extra)
            ctx.kept = kept
            ctx.save_for_backward(*tensors)
        elif checkpoint:
            with torch.no_grad():
                out = fn(*tensors, *extra)
            ctx.save_for_backward(*tensors)
        else:
            detached = [t.detach().requires_grad_(t.requires_grad) if t.is_floating_point() else t
                        for t in tensors]
            with torch.enable_grad():
                out = fn(*detached, *extra)
            ctx.detached, ctx.out = detached, out
            out = out.detach()
        engine._post_forward(unit_idx)
        return out

    @staticmethod
    def backward(ctx, dout):
        engine, u = ctx.engine, ctx.unit_idx
        engine._pre_backward(u)
        if ctx.checkpoint:
            tensors = [t.detach().requires_grad_(t.requires_grad) if t.is_floating_point() else t
                       for t in ctx.saved_tensors]
            with torch.enable_grad(), _ckpt.recompute(), \
                    (_ckpt.replay(ctx.kept) if ctx.kept is not None else contextlib.nullcontext()):
                out = ctx.fn(*tensors, *ctx.extra)
            ctx.kept = None
        else:
            tensors, out = ctx.detached, ctx.out
            ctx.detached = ctx.out = None
        torch.autograd.backward(out, dout)
        grads = tuple(t.grad if (t.is_floating_point() and t.requires_grad) else None for t in tensors)
        engine._post_backward(u)
        return (None, None, None, None, None) + grads + (None,) * len(ctx.extra)


class FSDPEngine:
    """Sharded trainer for models with ``embed_tokens(tokens)``, ``layers`` and ``head(x, targets)``.

    ``step(tokens, targets)`` runs forward, backward and the AdamW update and returns the loss
    tensor (on device).
    """

    def __init__(self, model: nn.Module, optim: AdamWConfig = AdamWConfig(),
                 group: Optional[dist.ProcessGroup] = None, comm: str = "auto",
                 activation_checkpointing: bool = True, max_grad_norm: Optional[float] = None,
                 unit_modules: Optional[Sequence[Sequence[nn.Module]]] = None,
                 layer_args: Callable[[nn.Module, Tensor], tuple] = None, symm_extra_bytes: int = 1 << 30,
                 replicate_group: Optional[dist.ProcessGroup] = None):
        self.model = model
        self.cfg = optim
        self.group = group
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        first = next(model.parameters())
        self.device = first.device
        self.param_dtype = first.dtype
        self.checkpoint = activation_checkpointing
        self.max_grad_norm = max_grad_norm
        # hybrid sharding (HSDP): parameters are sharded over `group` and replicated over
        # `replicate_group`; the reduced gradient shards are averaged over the replicas before the update
        self.replicate_group = replicate_group
        self.two_phase = max_grad_norm is not None or replicate_group is not None
        self.step_count = 0
        self.cuda = self.device.type == "cuda"
        if comm == "auto":
            comm = "single" if self.world == 1 else ("symm" if self.cuda else "torch")
        self.comm_kind = comm
        self.symm_extra_bytes = symm_extra_bytes
        self._build_units()
        self._alloc()
        self._dummy = torch.zeros(1, device=self.device, requires_grad=True)
        if self.cuda and self.world == 1:
            # the per-unit AdamW runs on a side stream under the next unit's backward: a small grid
            # that may share SMs with the persistent GEMM (TPB_ADAMW_OVERLAP="ctas_per_sm,max_shared")
            import os
            spec = os.environ.get("TPB_ADAMW_OVERLAP", "")
            if spec:
                c, m_ = (int(x) for x in spec.split(","))
                from .. import _native
                _native.kernels().tpb_adamw_set_overlap(c, m_)
        self.kernel_launch_estimate = 0
        self._status_host = None
        self._status_event = None

    # ------------------------------------------------------------------ construction
    def _build_units(self) -> None:
        m = self.model
        seen = set()

        def plist(named):
            out = []
            for n, p in named:
                if id(p) not in seen:
                    seen.add(id(p))
                    out.append((n, p))
            return out

        layer_params = [plist(layer.named_parameters(prefix=f"layers.{i}")) for i, layer in enumerate(m.layers)]
        layer_ids = {id(p) for lp in layer_params for _, p in lp}
        rest = [(n, p) for n, p in m.named_parameters() if id(p) not in layer_ids]
        embed_names = getattr(m, "embed_param_names", ("embed", "wte", "wpe", "tok_emb", "pos_emb"))
        emb = [(n, p) for n, p in rest if n.split(".")[0] in embed_names]
        head = [(n, p) for n, p in rest if n.split(".")[0] not in embed_names]
        groups = [("embed", emb)] + [(f"layer{i}", lp) for i, lp in enumerate(layer_params)] + [("head", head)]
        self.units: List[ParamUnit] = []
        for name, ps in groups:
            # expert-parallel parameters are owned by this rank alone: never gathered or reduced
            shared = [(n, p) for n, p in ps if not getattr(p, "_tpb_expert_parallel", False)]
            local = [(n, p) for n, p in ps if getattr(p, "_tpb_expert_parallel", False)]
            u = ParamUnit(len(self.units), name, shared, self.world, self.rank, self.device, self.param_dtype)
            u.local = ParamUnit(u.index, name + ".experts", local, 1, 0, self.device, self.param_dtype) if local else None
            self.units.append(u)
        self.n_layers = len(m.layers)

    def _alloc(self) -> None:
        dev, dt = self.device, self.param_dtype
        self.max_padded = max(u.padded for u in self.units)
        single = self.world == 1
        if self.comm_kind == "symm":
            from .symm import SymmComm
            self.comm = SymmComm(self, extra_bytes=self.symm_extra_bytes)
        else:
            self.comm = None
        for u in self.units:
            init = torch.zeros(u.padded, dtype=dt, device=dev)
            for (_, p), off, n in zip(u.params, u.offsets, u.numels):
                init[off: off + n].copy_(p.data.reshape(-1))
            lo, hi = u.shard_range()
            u.master = init[lo:hi].float()
            u.exp_avg = torch.zeros(u.shard_numel, dtype=torch.float32, device=dev)
            u.exp_avg_sq = torch.zeros(u.shard_numel, dtype=torch.float32, device=dev)
            if single:
                u.bind_params(init)
                u.shard = init
            else:
                u.shard = self.comm.alloc_shard(u) if self.comm is not None else init[lo:hi].clone()
                if self.comm is not None:
                    u.shard.copy_(init[lo:hi])
                # until gathered, parameters point at an empty placeholder
                for _, p in u.params:
                    p.data = torch.empty(0, dtype=dt, device=dev)
            del init
            if u.local is not None:
                lu = u.local
                full = torch.zeros(lu.padded, dtype=dt, device=dev)
                for (_, p), off, n in zip(lu.params, lu.offsets, lu.numels):
                    full[off: off + n].copy_(p.data.reshape(-1))
                lu.bind_params(full)
                lu.shard = full
                lu.master = full.float()
                lu.exp_avg = torch.zeros(lu.padded, dtype=torch.float32, device=dev)
                lu.exp_avg_sq = torch.zeros(lu.padded, dtype=torch.float32, device=dev)
        max_local = max([u.local.padded for u in self.units if u.local is not None] or [0])
        self.local_grad_pool = [torch.empty(max_local, dtype=dt, device=dev) for _ in range(2)] if max_local else []
        self.local_grad_events = [None, None]
        self._local_slot = 0
        # rotating full-parameter and gradient buffers
        # without checkpointing autograd keeps views of the gathered buffers until backward,
        # so every unit needs a buffer of its own for the whole step
        self.keep_gathered = not self.checkpoint
        n_full = 0 if single else (len(self.units) if self.keep_gathered else 3)
        n_grad = 2 if self.cuda else 2
        if self.comm is not None:
            self.full_pool = [self.comm.alloc_full(self.max_padded) for _ in range(n_full)]
            self.grad_pool = [self.comm.alloc_full(self.max_padded) for _ in range(n_grad)]
        else:
            self.full_pool = [torch.empty(self.max_padded, dtype=dt, device=dev) for _ in range(n_full)]
            self.grad_pool = [torch.empty(self.max_padded, dtype=dt, device=dev) for _ in range(n_grad)]
        self.grad_pool_events = [None] * n_grad
        self.full_owner = [None] * n_full
        if self.cuda:
            self.comm_stream = torch.cuda.Stream(device=dev)
            self.opt_stream = torch.cuda.Stream(device=dev)
        else:
            self.comm_stream = self.opt_stream = None
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.clip_coef = torch.ones(1, dtype=torch.float32, device=dev)
        self.grad_norm = torch.zeros(1, dtype=torch.float32, device=dev)  # last step's global norm
        self._grad_slot = 0

    # ------------------------------------------------------------------ gather / release
    def _gather(self, u: ParamUnit, slot: int) -> None:
        """Launch the all-gather of unit ``u`` into full-buffer ``slot`` on the comm stream."""
        buf = self.full_pool[slot][: u.padded]
        self.full_owner[slot] = u.index
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            if u.update_event is not None:
                self.comm_stream.wait_event(u.update_event)
            with torch.cuda.stream(self.comm_stream):
                self._gather_impl(u, buf)
                u.gather_event = torch.cuda.Event()
                u.gather_event.record(self.comm_stream)
        else:
            self._gather_impl(u, buf)
        u._slot = slot
        u._pending_full = buf

    def _gather_impl(self, u: ParamUnit, buf: Tensor) -> None:
        if self.comm is not None:
            self.comm.all_gather(u, buf)
        else:
            dist.all_gather_into_tensor(buf, u.shard, group=self.group)

    def _slot_for(self, u: ParamUnit) -> int:
        for i, owner in enumerate(self.full_owner):
            if owner == u.index:
                return i
        for i, owner in enumerate(self.full_owner):
            if owner is None:
                return i
        raise RuntimeError("no free full-parameter buffer")

    def _ensure_gathered(self, u: ParamUnit, prefetch: Optional[ParamUnit]) -> None:
        if self.world == 1:
            return
        if getattr(u, "_pending_full", None) is None:
            self._gather(u, self._slot_for(u))
        if self.cuda and u.gather_event is not None:
            torch.cuda.current_stream().wait_event(u.gather_event)
        u.bind_params(u._pending_full)
        if prefetch is not None and getattr(prefetch, "_pending_full", None) is None:
            try:
                self._gather(prefetch, self._slot_for(prefetch))
            except RuntimeError:
                pass  # all buffers busy; the gather happens when the unit is reached

    def _release(self, u: ParamUnit) -> None:
        if self.world == 1:
            return
        if self.cuda:
            # the buffer may be re-filled by the comm stream only after this unit's kernels ran
            u._release_event = torch.cuda.Event()
            u._release_event.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(u._release_event)
        self.full_owner[u._slot] = None
        u._pending_full = None
        u.full = None

    # ------------------------------------------------------------------ unit hooks
    def _pre_forward(self, idx: int) -> None:
        u = self.units[idx]
        nxt = self.units[idx + 1] if idx + 1 < len(self.units) else None
        self._ensure_gathered(u, nxt)

    def _post_forward(self, idx: int) -> None:
        u = self.units[idx]
        # the head's backward follows its forward immediately: keep it gathered
        if idx != len(self.units) - 1 and not self.keep_gathered:
            self._release(u)

    def _pre_backward(self, idx: int) -> None:
        u = self.units[idx]
        prv = self.units[idx - 1] if idx > 0 else None
        self._ensure_gathered(u, prv)
        slot = self._grad_slot
        self._grad_slot = (slot + 1) % len(self.grad_pool)
        ev = self.grad_pool_events[slot]
        if ev is not None and self.cuda:
            torch.cuda.current_stream().wait_event(ev)
        if self.comm is not None:
            self.comm.before_grad_reuse(slot)
        g = self.grad_pool[slot][: u.padded]
        u.zero_padding(g)
        u.bind_grads(g)
        u._grad_slot = slot
        if u.local is not None:
            ls = self._local_slot
            self._local_slot = (ls + 1) % 2
            ev = self.local_grad_events[ls]
            if ev is not None and self.cuda:
                torch.cuda.current_stream().wait_event(ev)
            lg = self.local_grad_pool[ls][: u.local.padded]
            u.local.zero_padding(lg)
            u.local.bind_grads(lg)
            u.local._grad_slot = ls

    def _post_backward(self, idx: int) -> None:
        u = self.units[idx]
        u.collect_autograd_grads()
        if u.local is not None:
            u.local.collect_autograd_grads()
        self._release(u)
        self._reduce_and_update(u)

    # ------------------------------------------------------------------ reduce + AdamW
    def _adam_kwargs(self):
        c = self.cfg
        return dict(lr=c.lr, beta1=c.betas[0], beta2=c.betas[1], eps=c.eps, weight_decay=c.weight_decay,
                    step=self.step_count)

    def _reduce_and_update(self, u: ParamUnit) -> None:
        g = u.grad
        stream = self.opt_stream if self.world == 1 else self.comm_stream
        if self.cuda:
            stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            if self.two_phase:
                self._reduce_only(u, g)
            elif self.world == 1:
                ops.adamw_flat_(u.master, u.exp_avg, u.exp_avg_sq, g, u.shard, **self._adam_kwargs())
            elif self.comm is not None:
                self.comm.reduce_scatter_adamw(u, g, self._adam_kwargs())
            else:
                gs = torch.empty(u.shard_numel, dtype=g.dtype, device=g.device)
                if g.device.type == "cpu" or dist.get_backend(self.group) == "gloo":
                    tmp = g.float()
                    dist.all_reduce(tmp, group=self.group)
                    lo, hi = u.shard_range()
                    gs = tmp[lo:hi].div_(self.world).to(g.dtype)
                else:
                    dist.reduce_scatter_tensor(gs, g, op=dist.ReduceOp.AVG, group=self.group)
                ops.adamw_flat_(u.master, u.exp_avg, u.exp_avg_sq, gs, u.shard, **self._adam_kwargs())
            if u.local is not None and self.two_phase:
                lu = u.local
                if lu.red is None:
                    lu.red = torch.empty(lu.padded, dtype=torch.float32, device=self.device)
                lu.red.copy_(lu.grad[: lu.padded]).mul_(1.0 / self.world)
                ops.sumsq_(lu.red, self.sumsq)
                if self.cuda:
                    lev = torch.cuda.Event()
                    lev.record(stream)
                    self.local_grad_events[lu._grad_slot] = lev
                lu.bind_grads(None)
            elif u.local is not None:
                lu = u.local
                ops.adamw_flat_(lu.master, lu.exp_avg, lu.exp_avg_sq, lu.grad, lu.shard,
                                grad_scale=1.0 / self.world, **self._adam_kwargs())
                if self.cuda:
                    lev = torch.cuda.Event()
                    lev.record(stream)
                    self.local_grad_events[lu._grad_slot] = lev
                    lu.update_event = lev
                lu.bind_grads(None)
            if self.cuda:
                ev = torch.cuda.Event()
                ev.record(stream)
                self.grad_pool_events[u._grad_slot] = ev
                u.update_event = ev
        u.bind_grads(None)

    # ------------------------------------------------------------------ gradient clipping (two phases)
    def _reduce_only(self, u: ParamUnit, g: Tensor) -> None:
        """Phase 1 of a clipped step: reduce this unit's gradient into its persistent shard-sized
        buffer and add its squared norm to the running total; the update waits for the global norm."""
        if u.red is None:
            dt = self.param_dtype if self.world == 1 else torch.float32
            u.red = torch.empty(u.shard_numel, dtype=dt, device=self.device)
        if self.world == 1:
            u.red.copy_(g[: u.shard_numel])
            ops.sumsq_(u.red, self.sumsq)
        elif self.comm is not None:
            self.comm.reduce_scatter_only(u, g, u.red, self.sumsq)
        else:
            if g.device.type == "cpu" or dist.get_backend(self.group) == "gloo":
                tmp = g.float()
                dist.all_reduce(tmp, group=self.group)
                lo, hi = u.shard_range()
                u.red.copy_(tmp[lo:hi]).div_(self.world)
            else:
                gs = torch.empty(u.shard_numel, dtype=g.dtype, device=g.device)
                dist.reduce_scatter_tensor(gs, g, op=dist.ReduceOp.AVG, group=self.group)
                u.red.copy_(gs)
            ops.sumsq_(u.red, self.sumsq)

    def _clipped_update(self) -> None:
        """Phase 2: global norm -> clip coefficient on the device -> AdamW on every shard."""
        stream = self.opt_stream if self.world == 1 else self.comm_stream
        if self.cuda:
            stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            if self.replicate_group is not None:
                # average the reduced shards over the replicas, then take the norm of the result
                r = dist.get_world_size(self.replicate_group)
                self.sumsq.zero_()
                for u in self.units:
                    if u.local is not None:
                        raise NotImplementedError("expert-parallel parameters are not supported with a replicate group")
                    if u.red.dtype == torch.float32 or u.red.device.type == "cuda":
                        dist.all_reduce(u.red, group=self.replicate_group)
                        u.red.div_(r)
                    else:
                        tmp = u.red.float()
                        dist.all_reduce(tmp, group=self.replicate_group)
                        u.red.copy_(tmp.div_(r))
                    ops.sumsq_(u.red, self.sumsq)
            clip = None
            if self.max_grad_norm is not None:
                if self.world > 1:
                    dist.all_reduce(self.sumsq, group=self.group)
                ops.clip_coef_(self.sumsq, float(self.max_grad_norm), self.clip_coef, self.grad_norm)
                clip = self.clip_coef
            kw = self._adam_kwargs()
            for u in self.units:
                for t in (u, u.local):
                    if t is None or t.red is None:
                        continue
                    ops.adamw_flat_(t.master, t.exp_avg, t.exp_avg_sq, t.red, t.shard, clip_coef=clip, **kw)
                    if self.cuda:
                        ev = torch.cuda.Event()
                        ev.record(stream)
                        t.update_event = ev
            self.sumsq.zero_()
        if self.cuda:
            # readers of grad_norm (and the next step) on the main stream see the finished update
            torch.cuda.current_stream().wait_stream(stream)

    # ------------------------------------------------------------------ public API
    def _poll_status(self, blocking: bool = False) -> None:
        """Raise ``DeviceWaitTimeout`` when a kernel of an earlier step gave up on a bounded wait.

        The status word is copied to pinned host memory at the end of every step without a
        synchronisation; the copy of step k is looked at when step k + 1 starts (or at once with
        ``blocking``), so training never continues silently on incomplete gradients."""
        if not self.cuda or self.comm is None:
            return
        from ..ops._common import DeviceWaitTimeout, status_word
        w = status_word(self.device)
        if self._status_host is None:
            self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        ev = self._status_event
        if ev is not None and (blocking or ev.query()):
            ev.synchronize()
            v = int(self._status_host[0]) & 0xFFFFFFFF
            if v:
                self._status_event = None
                w.zero_()
                names = {1: "mbarrier wait", 2: "flag wait", 3: "bad arguments"}
                raise DeviceWaitTimeout(
                    f"a communication kernel reported {names.get(v & 0xFF, v & 0xFF)} time-out at site {v >> 8}; "
                    "parameters of the affected units were left unchanged")

    def _record_status(self) -> None:
        if not self.cuda or self.comm is None:
            return
        from ..ops._common import status_word
        if self._status_host is None:
            self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        # read behind the communication stream's kernels of this step, without holding up compute
        with torch.cuda.stream(self.comm_stream):
            self._status_host.copy_(status_word(self.device), non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record(self.comm_stream)

    def forward_backward(self, tokens: Tensor, targets: Tensor) -> Tensor:
        m = self.model
        self._poll_status()
        self.step_count += 1
        if self.cuda:
            # parameters updated by the previous step's in-backward AdamW
            for u in self.units:
                if u.update_event is not None and self.world == 1:
                    torch.cuda.current_stream().wait_event(u.update_event)
                if u.local is not None and u.local.update_event is not None:
                    torch.cuda.current_stream().wait_event(u.local.update_event)
        x = _UnitFn.apply(self, 0, lambda d, t: m.embed_tokens(t), False, 1, self._dummy, tokens)
        extra = m.layer_extra_args(tokens) if hasattr(m, "layer_extra_args") else ()
        for i, layer in enumerate(m.layers):
            # each layer is a checkpointed region of its own: what it returns is the region's result
            layer._tpb_region_is_layer = True
            x = _UnitFn.apply(self, 1 + i, layer, self.checkpoint, 1, x, *extra)
        loss = _UnitFn.apply(self, len(self.units) - 1, lambda h, t: m.head(h, t), False, 1, x, targets)
        loss.backward()
        if self.two_phase:
            self._clipped_update()
        self._record_status()
        return loss.detach()

    def step(self, tokens: Tensor, targets: Tensor) -> Tensor:
        return self.forward_backward(tokens, targets)

    def synchronize(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            self._poll_status(blocking=True)

    # ------------------------------------------------------------------ checkpoint / resume
    def save_checkpoint(self, directory: str) -> None:
        """Sharded checkpoint: every rank writes its fp32 master / moment shards of every unit to
        ``rank{r}.mega`` (one collective-free file per rank); rank 0 adds ``engine.json`` with the
        layout. Expert-parallel (rank-local) parameters are stored whole in their owner's file."""
        import json
        import os
        from ..serialization import save
        os.makedirs(directory, exist_ok=True)
        self.synchronize()
        blob = {}
        for u in self.units:
            for tag, t in (("master", u.master), ("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq)):
                blob[f"{u.name}.{tag}"] = t.detach().cpu()
            if u.local is not None:
                for tag, t in (("master", u.local.master), ("exp_avg", u.local.exp_avg), ("exp_avg_sq", u.local.exp_avg_sq)):
                    blob[f"{u.name}.local.{tag}"] = t.detach().cpu()
        save(blob, os.path.join(directory, f"rank{self.rank}.mega"))
        if self.rank == 0:
            meta = {"world": self.world, "step": self.step_count,
                    "units": [{"name": u.name, "numel": u.numel, "padded": u.padded,
                               "params": [n for n, _ in u.params]} for u in self.units]}
            with open(os.path.join(directory, "engine.json"), "w") as f:
                json.dump(meta, f)
        if self.world > 1:
            dist.barrier(group=self.group)

    def load_checkpoint(self, directory: str) -> None:
        """Resume from :meth:`save_checkpoint`. The saving job may have had a different number of
        ranks: a unit's state is one flat vector cut into equal shards, so this rank's slice is
        assembled from the overlapping slices of the old shards."""
        import json
        import os
        from ..serialization import load
        with open(os.path.join(directory, "engine.json")) as f:
            meta = json.load(f)
        old_world = int(meta["world"])
        by_name = {m["name"]: m for m in meta["units"]}
        files = {}

        def old_file(r):
            if r not in files:
                files[r] = load(os.path.join(directory, f"rank{r}.mega"))
            return files[r]

        for u in self.units:
            m = by_name[u.name]
            if m["numel"] != u.numel or m["params"] != [n for n, _ in u.params]:
                raise ValueError(f"checkpoint unit {u.name} does not match the model")
            old_shard = int(m["padded"]) // old_world
            lo, hi = u.shard_range()
            for tag, dst in (("master", u.master), ("exp_avg", u.exp_avg), ("exp_avg_sq", u.exp_avg_sq)):
                out = torch.zeros(hi - lo, dtype=torch.float32)
                pos = lo
                while pos < min(hi, u.numel):
                    r = pos // old_shard
                    src = old_file(r)[f"{u.name}.{tag}"]
                    a = pos - r * old_shard
                    n = min(old_shard - a, min(hi, u.numel) - pos)
                    out[pos - lo: pos - lo + n] = src[a: a + n]
                    pos += n
                dst.copy_(out)
            u.shard.copy_(u.master[: u.shard.numel()] if self.world == 1 else u.master)
            if u.local is not None:
                if old_world != self.world:
                    raise ValueError("expert-parallel state cannot be resharded to another world size")
                src = old_file(self.rank)
                for tag, dst in (("master", u.local.master), ("exp_avg", u.local.exp_avg), ("exp_avg_sq", u.local.exp_avg_sq)):
                    dst.copy_(src[f"{u.name}.local.{tag}"])
                u.local.shard.copy_(u.local.master)
        self.step_count = int(meta["step"])
        if self.world > 1:
            dist.barrier(group=self.group)

    def gather_full_state(self) -> dict:
        """Full (unsharded) parameters as a name -> tensor dict on every rank (for checkpoints/tests)."""
        out = {}
        for u in self.units:
            if self.world == 1:
                full = u.master
            else:
                full = torch.empty(u.padded, dtype=torch.float32, device=self.device)
                if self.cuda:
                    torch.cuda.synchronize()
                dist.all_gather_into_tensor(full, u.master.contiguous(), group=self.group)
            for (n, p), off, cnt, shape in zip(u.params, u.offsets, u.numels, u.shapes):
                out[n] = full[off: off + cnt].view(shape).clone()
            if u.local is not None:
                lu = u.local
                for (n, p), off, cnt, shape in zip(lu.params, lu.offsets, lu.numels, lu.shapes):
                    out[n] = lu.master[off: off + cnt].view(shape).clone()
        return out
