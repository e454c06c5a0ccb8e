"""DistributedDataParallel with a bucketed reducer overlapped with backward.

Gradients live as views of flat 25 MiB buckets (built in reverse parameter order, the order
backward produces them); a post-accumulate hook counts a bucket's parameters down and launches
its reduction on a communication stream as soon as the bucket is complete. Three reduction paths:

* ``torch`` collectives (gloo / NCCL all-reduce) - the baseline and the CPU path;
* ``symm``: in-place all-reduce over peer memory (each rank reduces its slice of the bucket in
  fp32 and stores the bf16 result into every peer's bucket);
* ``symm`` + ``fused_adamw``: the same kernel also applies AdamW to the slice it owns and
  broadcasts the new bf16 parameters into every rank's parameter bucket, so that
  ``optimizer.step()`` disappears (ZeRO-1 style sharded optimizer state).

Replaces the reference's C++ ``DDPReducer`` (src/bindings/python/Distributed.cpp:33-247:
eager copy-in, in-order flush, ncclAllReduce on a pooled stream) and its Python wrapper
(tensorplay/nn/parallel/distributed.py:265-400, ``no_sync`` :824-836).
"""
from __future__ import annotations

import contextlib
from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.engine import AdamWConfig
from .algorithms.join import Join, Joinable, JoinHook
from .. import ops


class _Bucket:
    def __init__(self, index: int, params: List[nn.Parameter], flat_grad: torch.Tensor,
                 flat_param: Optional[torch.Tensor]):
        self.index, self.params = index, params
        self.flat_grad, self.flat_param = flat_grad, flat_param
        self.event = None


class GradBucket:
    """What a communication hook receives (tensorplay/distributed/distributed_core.py:3325-3358)."""

    def __init__(self, b: _Bucket, last: bool):
        self._b, self._last = b, last

    def index(self): return self._b.index
    def buffer(self): return self._b.flat_grad
    def set_buffer(self, t): self._b.flat_grad.copy_(t)
    def gradients(self): return [p.grad for p in self._b.params]
    def parameters(self): return self._b.params
    def is_last(self): return self._last


class _DDPJoinHook(JoinHook):
    """A rank without inputs left answers one iteration of the others: the buffer broadcasts of their
    forward and every bucket's reduction, in bucket order, with zero gradients (the average still divides
    by the full world size). Afterwards the parameters of a rank that trained to the end are published."""

    def __init__(self, ddp: "DistributedDataParallel"):
        self.ddp = ddp

    def main_hook(self) -> None:
        d = self.ddp
        if d.broadcast_buffers and d.world > 1:
            for buf in d.module.buffers():
                dist.broadcast(buf, src=0, group=d.process_group)
        for b in d.buckets:
            b.flat_grad.zero_()
            d._reduce(b)
        d.synchronize()

    def post_hook(self, is_last_joiner: bool) -> None:
        d = self.ddp
        who = torch.tensor([d.rank if is_last_joiner else -1], device=d.device)
        dist.all_reduce(who, op=dist.ReduceOp.MAX, group=d.process_group)
        src = int(who.item())
        src = dist.get_global_rank(d.process_group, src) if d.process_group is not None else src
        for t in list(d.module.parameters()) + list(d.module.buffers()):
            dist.broadcast(t.data, src=src, group=d.process_group)


class DistributedDataParallel(nn.Module, Joinable):
    def __init__(self, module: nn.Module, device_ids=None, output_device=None, dim: int = 0,
                 broadcast_buffers: bool = True, process_group=None, bucket_cap_mb: float = 25.0,
                 find_unused_parameters: bool = False, gradient_as_bucket_view: bool = True,
                 static_graph: bool = False, comm: str = "auto",
                 fused_adamw: Optional[AdamWConfig] = None):
        super().__init__()
        Joinable.__init__(self)
        self.module = module
        self.process_group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.broadcast_buffers = broadcast_buffers
        # Parameters that take no part in a backward never fire their hook, so their bucket would never
        # fill. With find_unused_parameters the buckets that are still open when the backward ends are
        # completed with zeros for those parameters and reduced; without it an open bucket is an error
        # (it would otherwise skip its reduction silently). static_graph needs nothing here: readiness
        # is counted by hooks on the parameters, not discovered from the autograd graph.
        self.find_unused_parameters = find_unused_parameters
        self.static_graph = static_graph
        if device_ids is not None:
            if len(device_ids) != 1:
                raise ValueError("device_ids must name exactly one device: one process drives one GPU")
            want = device_ids[0] if isinstance(device_ids[0], int) else torch.device(device_ids[0]).index
            have = next(module.parameters()).device
            if have.type != "cuda" or have.index != want:
                raise ValueError(f"the module lives on {have}, device_ids says cuda:{want}; move the module first")
        if output_device is not None and device_ids is not None and output_device != device_ids[0]:
            raise NotImplementedError("output_device other than the module's device is not implemented")
        if dim != 0:
            raise NotImplementedError("scattering inputs along a dimension (dim) is not implemented: pass each rank its batch")
        self._ready_in_bucket = {}
        self._reduced = set()
        self._complete = set()
        self._next_bucket = 0
        self._cb_queued = False
        self.require_backward_grad_sync = True
        self._hook = None
        self._hook_state = None
        params = [p for p in module.parameters() if p.requires_grad]
        self.device = params[0].device
        self.cuda = self.device.type == "cuda"
        if comm == "auto":
            comm = "symm" if (self.cuda and self.world > 1 and params[0].dtype == torch.bfloat16) else "torch"
        self.comm_kind = comm
        self.fused = fused_adamw
        if self.fused is not None and comm != "symm" and self.world > 1:
            raise ValueError("fused_adamw needs the symmetric-memory path (bf16 parameters on CUDA)")
        self._sync_module_states()
        self._build_buckets(params, int(bucket_cap_mb * 1024 * 1024))
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self.step_count = 0
        self._accum = False
        for p in params:
            p.register_post_accumulate_grad_hook(self._make_hook(p))

    # ---------------------------------------------------------------- construction
    def _sync_module_states(self) -> None:
        if self.world == 1:
            return
        with torch.no_grad():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                dist.broadcast(t.data, src=dist.get_global_rank(self.process_group, 0) if self.process_group else 0,
                               group=self.process_group)

    def _build_buckets(self, params, cap_bytes) -> None:
        # bucket assignment and ready counting live in the native reducer (csrc/runtime/reducer.cpp)
        import ctypes as C
        from .. import _native
        rt = _native.runtime()
        rt.tpb_reducer_create.restype = C.c_void_p
        rt.tpb_reducer_create.argtypes = [C.POINTER(C.c_longlong), C.POINTER(C.c_int), C.c_int, C.c_longlong,
                                          C.c_longlong]
        for fn, res, args in (("tpb_reducer_num_buckets", C.c_int, [C.c_void_p]),
                              ("tpb_reducer_bucket_size", C.c_int, [C.c_void_p, C.c_int]),
                              ("tpb_reducer_bucket_numel", C.c_longlong, [C.c_void_p, C.c_int]),
                              ("tpb_reducer_offset_of", C.c_longlong, [C.c_void_p, C.c_int]),
                              ("tpb_reducer_bucket_members", None, [C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
                              ("tpb_reducer_mark_ready", C.c_int, [C.c_void_p, C.c_int]),
                              ("tpb_reducer_rearm", None, [C.c_void_p, C.c_int]),
                              ("tpb_reducer_reset", None, [C.c_void_p]),
                              ("tpb_reducer_destroy", None, [C.c_void_p])):
            f = getattr(rt, fn)
            f.restype, f.argtypes = res, args
        n = len(params)
        self._rt = rt
        self._reducer = rt.tpb_reducer_create((C.c_longlong * n)(*[p.numel() for p in params]),
                                              (C.c_int * n)(*[p.element_size() for p in params]), n,
                                              int(cap_bytes), self.world * 128)
        self._param_index = {id(p): i for i, p in enumerate(params)}
        groups = []
        for b in range(rt.tpb_reducer_num_buckets(self._reducer)):
            m = (C.c_int * rt.tpb_reducer_bucket_size(self._reducer, b))()
            rt.tpb_reducer_bucket_members(self._reducer, b, m)
            groups.append([params[i] for i in m])
        arena = None
        if self.comm_kind == "symm":
            from ..parallel.symm import SymmArena
            esz = params[0].element_size()
            total = sum(((sum((p.numel() + 7) // 8 * 8 for p in g) + self.world * 128 - 1) // (self.world * 128)) * self.world * 128
                        for g in groups) * esz * 2 + (1 << 22)
            arena = SymmArena._instance or SymmArena(total + (8 << 20), group=self.process_group)
        self.arena = arena
        self.buckets: List[_Bucket] = []
        self._bucket_of = {}
        for gi, g in enumerate(groups):
            offs = [int(self._rt.tpb_reducer_offset_of(self._reducer, self._param_index[id(p)])) for p in g]
            padded = int(self._rt.tpb_reducer_bucket_numel(self._reducer, gi))
            if arena is not None:
                fg = arena.alloc(padded, g[0].dtype)
                fp = arena.alloc(padded, g[0].dtype)
                fg.zero_()
            else:
                fg = torch.zeros(padded, dtype=g[0].dtype, device=self.device)
                fp = None
            b = _Bucket(gi, g, fg, fp)
            b.offsets, b.padded = offs, padded
            b.offset_of = {id(p): o for p, o in zip(g, offs)}
            for p, o in zip(g, offs):
                if fp is not None:
                    fp[o: o + p.numel()].copy_(p.data.reshape(-1))
                    p.data = fp[o: o + p.numel()].view(p.shape)
                p.grad = fg[o: o + p.numel()].view(p.shape)
                self._bucket_of[id(p)] = b
            if arena is not None:
                w = self.world
                b.slot_ready, b.slot_done = arena.slots(w), arena.slots(w)
                b.epoch = 0
                if self.fused is not None:
                    shard = padded // w
                    lo = self.rank * shard
                    b.master = fp[lo: lo + shard].float()
                    b.exp_avg = torch.zeros(shard, dtype=torch.float32, device=self.device)
                    b.exp_avg_sq = torch.zeros(shard, dtype=torch.float32, device=self.device)
            self.buckets.append(b)

    # ---------------------------------------------------------------- reduction
    def _make_hook(self, p):
        def hook(param):
            if not self.require_backward_grad_sync or self.world == 1 and self.fused is None:
                return
            b = self._bucket_of[id(param)]
            o = b.offset_of[id(param)]
            v = b.flat_grad[o: o + param.numel()]
            if param.grad.data_ptr() != v.data_ptr():
                v.copy_(param.grad.reshape(-1))
                param.grad = v.view(param.shape)
            if not self._cb_queued:
                self._cb_queued = True
                torch.autograd.Variable._execution_engine.queue_callback(self._finalize_backward)
            self._ready_in_bucket.setdefault(b.index, set()).add(id(param))
            done = self._rt.tpb_reducer_mark_ready(self._reducer, self._param_index[id(param)])
            if done >= 0:
                self._complete.add(done)
                self._launch_in_order()
        return hook

    def _launch_in_order(self) -> None:
        """Reductions are issued strictly in bucket order (the order in which a full backward fills
        them): ranks whose buckets fill in different orders - some parameters unused on some ranks -
        still issue the same sequence of collectives."""
        while self._next_bucket < len(self.buckets) and self._next_bucket in self._complete:
            b = self.buckets[self._next_bucket]
            self._next_bucket += 1
            self._reduced.add(b.index)
            self._reduce(b)

    def _finalize_backward(self) -> None:
        """End of a synchronised backward: every bucket must have been reduced."""
        ready, reduced, complete = self._ready_in_bucket, self._reduced, self._complete
        self._ready_in_bucket, self._reduced, self._complete, self._cb_queued = {}, set(), set(), False
        self._next_bucket = 0
        open_buckets = [b for b in self.buckets if b.index not in reduced]
        if not open_buckets:
            return
        if not self.find_unused_parameters:
            for b in open_buckets:
                self._rt.tpb_reducer_rearm(self._reducer, b.index)
            names = {id(p): n for n, p in self.module.named_parameters()}
            missing = [names.get(id(p), "?") for b in open_buckets for p in b.params if id(p) not in ready.get(b.index, ())]
            raise RuntimeError("DistributedDataParallel: these parameters received no gradient in this backward, so "
                               f"their buckets were not reduced: {missing[:8]}{' ...' if len(missing) > 8 else ''}. "
                               "Pass find_unused_parameters=True if parts of the model are skipped on purpose.")
        for b in open_buckets:   # ascending bucket order, after everything that was launched during the backward
            got = ready.get(b.index, ())
            for p in b.params:
                if id(p) not in got:
                    o = b.offset_of[id(p)]
                    b.flat_grad[o: o + p.numel()].zero_()   # unused this step: contributes zeros to the average
            if b.index not in complete:
                self._rt.tpb_reducer_rearm(self._reducer, b.index)
            self._reduce(b)

    def _reduce(self, b: _Bucket) -> None:
        last = b.index == len(self.buckets) - 1
        if self._hook is not None:
            fut = self._hook(self._hook_state, GradBucket(b, last))
            out = fut.wait() if hasattr(fut, "wait") else fut
            out = out[0] if isinstance(out, (list, tuple)) else out
            if out is not None and out.data_ptr() != b.flat_grad.data_ptr():
                b.flat_grad.copy_(out)
            self._rt.tpb_reducer_rearm(self._reducer, b.index)
            return
        if self.cuda:
            self.comm_stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(self.comm_stream)
        else:
            ctx = contextlib.nullcontext()
        with ctx:
            if self.comm_kind == "symm" and self.world >= 1 and self.arena is not None:
                self._reduce_symm(b)
            elif self.world > 1:
                if b.flat_grad.dtype == torch.float32 or dist.get_backend(self.process_group) == "gloo":
                    dist.all_reduce(b.flat_grad, group=self.process_group)
                    b.flat_grad.div_(self.world)
                else:
                    dist.all_reduce(b.flat_grad, op=dist.ReduceOp.AVG, group=self.process_group)
            if self.cuda:
                b.event = torch.cuda.Event()
                b.event.record(self.comm_stream)
        self._rt.tpb_reducer_rearm(self._reducer, b.index)

    def _reduce_symm(self, b: _Bucket) -> None:
        from .. import _native
        from ..ops._common import status_word, stream_ptr
        from ..parallel.symm import NO_OFFSET
        a = self.arena
        b.epoch += 1
        shard = b.padded // self.world
        lo = self.rank * shard
        goff = a.offset_of(b.flat_grad)
        st = status_word(self.device)
        if self.fused is not None:
            c = self.fused
            code = a.raw.tpb_symm_rs_adamw(
                goff, lo, shard, b.master.data_ptr(), b.exp_avg.data_ptr(), b.exp_avg_sq.data_ptr(), None,
                a.offset_of(b.flat_param), None, None, 0, c.lr, c.betas[0], c.betas[1], c.eps, c.weight_decay,
                self.step_count + 1, 1.0 / self.world, None, a.pad_off, b.slot_ready, b.slot_done, b.epoch,
                a.counter_ptr(b.index), 64, 30.0, st.data_ptr(), stream_ptr())
        else:
            code = a.raw.tpb_symm_rs_adamw(
                goff, lo, shard, None, None, None, None, goff, None, None, 2, 0.0, 0.0, 0.0, 0.0, 0.0, 1,
                1.0 / self.world, None, a.pad_off, b.slot_ready, b.slot_done, b.epoch,
                a.counter_ptr(b.index), 64, 30.0, st.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_rs_adamw")
        # every rank's slice must have landed before this rank reads the bucket again
        code = a.raw.tpb_symm_wait_slots(a.pad_off, b.slot_done, b.epoch, 30.0, st.data_ptr(), stream_ptr())
        _native.launch_count += 1
        _native.check(code, "tpb_symm_wait_slots")

    # ---------------------------------------------------------------- module API
    def forward(self, *args, **kwargs):
        if self.require_backward_grad_sync:
            Join.notify_join_context(self)
        if self.cuda:
            for b in self.buckets:
                if b.event is not None:
                    torch.cuda.current_stream().wait_event(b.event)
        if self.broadcast_buffers and self.world > 1 and self.require_backward_grad_sync:
            for buf in self.module.buffers():
                dist.broadcast(buf, src=0, group=self.process_group)
        return self.module(*args, **kwargs)

    def finish_step(self) -> None:
        """With ``fused_adamw``: call after ``backward`` instead of ``optimizer.step()`` +
        ``zero_grad()``. Orders the main stream after the reductions and clears the buckets."""
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        self.step_count += 1
        for b in self.buckets:
            b.flat_grad.zero_()

    def synchronize(self) -> None:
        """Order the current stream after all outstanding bucket reductions."""
        if self.cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)

    # ---------------------------------------------------------------- uneven inputs
    def join(self, divide_by_initial_world_size: bool = True, enable: bool = True,
             throw_on_early_termination: bool = False):
        """Context manager for training with a different number of batches per rank
        (tensorplay/nn/parallel/distributed.py ``join``). Gradients are always averaged over the full
        world size."""
        if not divide_by_initial_world_size:
            raise NotImplementedError("dividing by the number of ranks still training is not implemented")
        return Join([self], enable, throw_on_early_termination)

    def join_hook(self, **kwargs) -> JoinHook:
        return _DDPJoinHook(self)

    @property
    def join_device(self) -> torch.device:
        return self.device

    @property
    def join_process_group(self):
        return self.process_group if self.process_group is not None else dist.group.WORLD

    @contextlib.contextmanager
    def no_sync(self):
        old = self.require_backward_grad_sync
        self.require_backward_grad_sync = False
        try:
            yield
        finally:
            self.require_backward_grad_sync = old

    def register_comm_hook(self, state, hook) -> None:
        """``hook(state, bucket: GradBucket) -> Future[Tensor] | Tensor``."""
        self._hook_state, self._hook = state, hook

    def state_dict(self, *a, **kw):
        return self.module.state_dict(*a, **kw)

    def load_state_dict(self, *a, **kw):
        return self.module.load_state_dict(*a, **kw)
