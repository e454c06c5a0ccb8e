"""Tensor / sequence parallel linears on the fused compute+collective kernels.

``AllGatherLinear``  : y = all_gather_rows(x_local) @ W_shard^T   (column-parallel: QKV, gate/up)
``LinearReduceScatter``: y_local = reduce_scatter_rows(x @ W_shard^T) (row-parallel: o_proj, down)

Forward and backward are each ONE kernel launch that moves the activations over NVLink peer
memory while the tcgen05 tiles run (copy CTAs + per-chunk flags for the gather; P2P epilogue
stores + arrival counters for the scatter). The backward of one is the other:
  d(all-gather -> GEMM)      : dx_local = reduce_scatter(dy @ W),  dW = dy^T @ x_full
  d(GEMM -> reduce-scatter)  : dx = all_gather(dy_local) @ W,      dW = dy_full^T @ x
The reference composes these from DTensor redistributes around cuBLAS
(tensorplay/distributed/tensor/parallel/style.py:67-176 -> funcol all_gather_single /
reduce_scatter_single, _functional_collectives.py:569-638).
On CPU ranks (gloo) the same functions run as plain collectives + matmul.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native, ops
from ..ops._common import status_word, stream_ptr
from .symm import SymmArena

_SIGS = {
    "tpb_ag_gemm": [C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                    C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int,
                    C.c_uint32, C.c_int, C.c_double, C.c_void_p, C.c_void_p, C.c_void_p],
    "tpb_ag_gemm_weight": [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                           C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_size_t, C.c_int, C.c_int,
                           C.c_uint32, C.c_int, C.c_double, C.c_void_p, C.c_void_p, C.c_void_p],
    "tpb_symm_allreduce_residual_norm": [C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float,
                                         C.c_size_t, C.c_int, C.c_void_p, C.c_void_p, C.c_double, C.c_void_p,
                                         C.c_void_p],
    "tpb_gemm_rs": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                    C.c_int, C.c_int, C.c_size_t, C.c_size_t, C.c_int, C.c_uint32, C.c_double,
                    C.c_void_p, C.c_void_p, C.c_void_p],
    "tpb_symm_wait_slots_dev": [C.c_size_t, C.c_int, C.c_void_p, C.c_double, C.c_void_p, C.c_void_p],
    "tpb_symm_bump": [C.c_void_p, C.c_void_p],
}


def _raw(arena):
    raw = arena.raw
    if not getattr(raw, "_tp_sigs", False):
        _native.register_sigs(raw, _SIGS)
        raw._tp_sigs = True
    return raw


class AGGemmPlan:
    """Buffers and signal slots for all-gather(rows) -> GEMM with a fixed [M_total, K]."""

    def __init__(self, arena: SymmArena, m_total: int, k: int, rows_per_flag: int = 128,
                 n_copy: int = 16, wait_s: float = 30.0):
        w = arena.world
        assert m_total % w == 0 and (m_total // w) % rows_per_flag == 0
        self.arena, self.m, self.k, self.world, self.rank = arena, m_total, k, w, arena.rank
        self.rows = m_total // w
        self.rpf, self.n_copy, self.wait_s = rows_per_flag, n_copy, wait_s
        self.full = [arena.alloc(m_total * k, torch.bfloat16).view(m_total, k) for _ in range(2)]
        self.flags = [torch.zeros(w * (self.rows // rows_per_flag) + 1, dtype=torch.int32, device=arena.device)
                      for _ in range(2)]
        self.ready = [arena.slots(w) for _ in range(2)]
        self.done = [arena.slots(w) for _ in range(2)]
        # Epochs live on the device (one word per buffer, bumped in stream order after each launch):
        # no host-side counter enters a launch, so a sequence of calls can be replayed from a CUDA graph.
        self.epoch_dev = torch.zeros(2, dtype=torch.int32, device=arena.device)
        self.calls = 0
        self.status = status_word(arena.device)

    def local_view(self) -> torch.Tensor:
        """Where this rank's rows of the next call go (write here, then call ``run``)."""
        i = self.calls & 1
        raw = _raw(self.arena)
        if self.world > 1:
            # peers must have finished pulling the previous contents of this buffer
            _native.check(raw.tpb_symm_wait_slots_dev(self.arena.pad_off, self.done[i], self.epoch_dev[i:].data_ptr(),
                                                      self.wait_s, self.status.data_ptr(), stream_ptr()),
                          "tpb_symm_wait_slots_dev")
            _native.launch_count += 1
        return self.full[i][self.rank * self.rows: (self.rank + 1) * self.rows]

    def run(self, weight: torch.Tensor, bias=None, b_mn: bool = False, out=None):
        """C[M_total, N] = gathered_rows @ weight^T; returns (C, gathered rows)."""
        i = self.calls & 1
        self.calls += 1
        n = weight.shape[1] if b_mn else weight.shape[0]
        if out is None:
            out = torch.empty(self.m, n, dtype=torch.bfloat16, device=weight.device)
        raw = _raw(self.arena)
        code = raw.tpb_ag_gemm(self.arena.offset_of(self.full[i]), weight.data_ptr(), out.data_ptr(),
                               None if bias is None else bias.data_ptr(), self.m, n, self.k, weight.stride(0),
                               out.stride(0), int(b_mn), 0, self.flags[i].data_ptr(), self.rpf,
                               self.arena.pad_off, self.ready[i], self.done[i], 0, self.n_copy,
                               self.wait_s, self.status.data_ptr(), stream_ptr(), self.epoch_dev[i:].data_ptr())
        _native.check(code, "tpb_ag_gemm")
        _native.check(raw.tpb_symm_bump(self.epoch_dev[i:].data_ptr(), stream_ptr()), "tpb_symm_bump")
        _native.launch_count += 2
        return out, self.full[i]


class WeightAGGemmPlan:
    """A fully sharded weight ``[N, K]`` (rank ``r`` owns rows ``[r N / world, (r + 1) N / world)``) gathered INSIDE
    the GEMM that consumes it: ``C[M, N] = x[M, K] @ gather(W)^T``. Copy CTAs of the launch pull the peers' shards
    into the local full buffer while the tensor-core CTAs begin with the tiles of the local rows; after the call
    the full weight is resident for the other uses of the unit (the fused form of an FSDP all-gather followed by
    the first GEMM of the unit; the reference runs copy-in, ``all_gather_single``, copy-out before the GEMM,
    tensorplay/distributed/fsdp/_fully_shard/_fsdp_collectives.py:337-470)."""

    def __init__(self, arena: SymmArena, n_total: int, k: int, rows_per_flag: int = 256, n_copy: int = 16,
                 wait_s: float = 30.0):
        w = arena.world
        assert n_total % w == 0 and (n_total // w) % rows_per_flag == 0
        self.arena, self.n, self.k, self.world, self.rank = arena, n_total, k, w, arena.rank
        self.rows = n_total // w
        self.rpf, self.n_copy, self.wait_s = rows_per_flag, n_copy, wait_s
        self.full = arena.alloc(n_total * k, torch.bfloat16).view(n_total, k)
        self.flags = torch.zeros(w * (self.rows // rows_per_flag) + 1, dtype=torch.int32, device=arena.device)
        self.ready, self.done = arena.slots(w), arena.slots(w)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=arena.device)
        self.status = status_word(arena.device)

    def shard_view(self) -> torch.Tensor:
        """This rank's rows of the full buffer: the shard lives here (peers read it from this place)."""
        return self.full[self.rank * self.rows: (self.rank + 1) * self.rows]

    def wait_readers(self) -> None:
        """Order the stream after every peer's reads of this rank's shard in the previous call (call before
        the shard is rewritten, e.g. by the optimizer step)."""
        if self.world > 1:
            raw = _raw(self.arena)
            _native.check(raw.tpb_symm_wait_slots_dev(self.arena.pad_off, self.done, self.epoch_dev.data_ptr(),
                                                      self.wait_s, self.status.data_ptr(), stream_ptr()),
                          "tpb_symm_wait_slots_dev")
            _native.launch_count += 1

    def run(self, x: torch.Tensor, bias=None, out=None) -> torch.Tensor:
        m = x.shape[0]
        if out is None:
            out = torch.empty(m, self.n, dtype=torch.bfloat16, device=x.device)
        raw = _raw(self.arena)
        code = raw.tpb_ag_gemm_weight(x.data_ptr(), self.arena.offset_of(self.full), out.data_ptr(),
                                      None if bias is None else bias.data_ptr(), m, self.n, self.k, x.stride(0),
                                      out.stride(0), 0, 0, self.flags.data_ptr(), self.rpf, self.arena.pad_off,
                                      self.ready, self.done, 0, self.n_copy, self.wait_s, self.status.data_ptr(),
                                      stream_ptr(), self.epoch_dev.data_ptr())
        _native.check(code, "tpb_ag_gemm_weight")
        _native.check(raw.tpb_symm_bump(self.epoch_dev.data_ptr(), stream_ptr()), "tpb_symm_bump")
        _native.launch_count += 2
        return out


class AllReduceNormPlan:
    """Row-parallel outputs of a small batch (decode): every rank writes its partial ``[rows, H]`` product into
    ``partial()`` (an arena slice, e.g. as the ``out=`` of the GEMM), then ``run(x, norm_w, eps)`` adds the sum over
    ranks to the replicated residual stream ``x`` in place and returns ``rmsnorm(x) * norm_w`` for the next
    projection: all-reduce, residual add and norm in one launch, the sum taken inside the switch where the arena
    has a multicast mapping. The two partial slices alternate from call to call, which is what makes a closing
    rendezvous unnecessary; the epoch lives on the device, so the call sequence can be replayed from a CUDA
    graph. (The reference's row-parallel linear is an NCCL all-reduce after the GEMM,
    tensorplay/distributed/tensor/parallel/style.py ``RowwiseParallel``.)"""

    def __init__(self, arena: SymmArena, rows: int, hidden: int, wait_s: float = 30.0):
        self.arena, self.rows, self.H, self.wait_s = arena, rows, hidden, wait_s
        self.bufs = [arena.alloc(rows * hidden, torch.bfloat16).view(rows, hidden) for _ in range(2)]
        self.slot = arena.slots(arena.world)
        self.epoch_dev = torch.zeros(1, dtype=torch.int32, device=arena.device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=arena.device)
        self.calls = 0
        self.status = status_word(arena.device)

    def partial(self) -> torch.Tensor:
        """Where the partial of the next ``run`` goes."""
        return self.bufs[self.calls & 1]

    def run(self, x: torch.Tensor, norm_w: Optional[torch.Tensor] = None, eps: float = 1e-5,
            h_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        buf = self.bufs[self.calls & 1]
        self.calls += 1
        rows = x.shape[0]
        assert rows <= self.rows and x.shape[1] == self.H and x.is_contiguous()
        if norm_w is not None and h_out is None:
            h_out = torch.empty_like(x)
        raw = _raw(self.arena)
        code = raw.tpb_symm_allreduce_residual_norm(
            self.arena.offset_of(buf), x.data_ptr(), None if norm_w is None else norm_w.data_ptr(),
            None if h_out is None else h_out.data_ptr(), rows, self.H, float(eps), self.arena.pad_off, self.slot,
            self.epoch_dev.data_ptr(), self.counter.data_ptr(), self.wait_s, self.status.data_ptr(), stream_ptr())
        _native.check(code, "tpb_symm_allreduce_residual_norm")
        _native.launch_count += 1
        return h_out


class GemmRSPlan:
    """Buffers and counters for GEMM -> reduce-scatter(rows) with a fixed [M_total, N]."""

    def __init__(self, arena: SymmArena, m_total: int, n: int, wait_s: float = 30.0):
        w = arena.world
        assert m_total % w == 0 and n % 8 == 0
        self.arena, self.m, self.n, self.world, self.rank = arena, m_total, n, w, arena.rank
        self.rows = m_total // w
        self.stage = [arena.alloc(m_total * n, torch.bfloat16) for _ in range(2)]
        self.cnt = [arena.slots(w) for _ in range(2)]
        self.epoch_dev = torch.zeros(2, dtype=torch.int32, device=arena.device)  # see AGGemmPlan
        self.calls = 0
        self.wait_s = wait_s
        self.status = status_word(arena.device)

    def run(self, a: torch.Tensor, weight: torch.Tensor, a_mn: bool = False, b_mn: bool = False, out=None):
        """out[M_total / world, N] = rows of this rank of sum_r (A_r @ W_r^T)."""
        i = self.calls & 1
        self.calls += 1
        k = a.shape[0] if a_mn else a.shape[1]
        if out is None:
            out = torch.empty(self.rows, self.n, dtype=torch.bfloat16, device=a.device)
        raw = _raw(self.arena)
        code = raw.tpb_gemm_rs(a.data_ptr(), weight.data_ptr(), out.data_ptr(), self.m, self.n, k, a.stride(0),
                               weight.stride(0), int(a_mn), int(b_mn), self.arena.offset_of(self.stage[i]),
                               self.arena.pad_off, self.cnt[i], 0, self.wait_s,
                               self.status.data_ptr(), stream_ptr(), self.epoch_dev[i:].data_ptr())
        _native.check(code, "tpb_gemm_rs")
        _native.check(raw.tpb_symm_bump(self.epoch_dev[i:].data_ptr(), stream_ptr()), "tpb_symm_bump")
        _native.launch_count += 2
        return out


class _AGLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, weight, ag_plan: AGGemmPlan, rs_plan: Optional[GemmRSPlan]):
        ag_plan.local_view().copy_(x_local.reshape(-1, x_local.shape[-1]))
        y, x_full = ag_plan.run(weight)
        # the gathered rows live in the plan's rotating buffer, which the next calls of the same
        # shape overwrite: backward gets its own copy (needed for dW only)
        keep = x_full.clone() if weight.requires_grad else x_full.new_empty(0)
        ctx.save_for_backward(keep, weight)
        ctx.rs_plan = rs_plan
        ctx.w_ref = weight if hasattr(weight, "_tpb_grad_view") else None
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, weight = ctx.saved_tensors
        dy = dy.contiguous()
        # dx_local = reduce_scatter(dy @ W)
        dx = ctx.rs_plan.run(dy, weight, b_mn=True)
        w_ref = ctx.w_ref
        if not ctx.needs_input_grad[1]:
            return dx, None, None, None
        if w_ref is not None and w_ref._tpb_grad_view is not None:
            ops.gemm(dy, x_full, a_mn=True, b_mn=True, out=w_ref._tpb_grad_view,
                     accumulate=getattr(w_ref, "_tpb_grad_written", False))
            w_ref._tpb_grad_written = True
            dw = None
        else:
            dw = ops.gemm(dy, x_full, a_mn=True, b_mn=True)
        return dx, dw, None, None


class _LinearRSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, rs_plan: GemmRSPlan, ag_plan: Optional[AGGemmPlan]):
        x2 = x.reshape(-1, x.shape[-1])
        y = rs_plan.run(x2, weight)
        ctx.save_for_backward(x2, weight)
        ctx.ag_plan = ag_plan
        ctx.w_ref = weight if hasattr(weight, "_tpb_grad_view") else None
        return y

    @staticmethod
    def backward(ctx, dy_local):
        x2, weight = ctx.saved_tensors
        plan = ctx.ag_plan
        plan.local_view().copy_(dy_local.reshape(-1, dy_local.shape[-1]))
        # dx = all_gather(dy_local) @ W   (W stored [N_out, K_in]: B operand is MN-major)
        dx, dy_full = plan.run(weight, b_mn=True)
        w_ref = ctx.w_ref
        if w_ref is not None and w_ref._tpb_grad_view is not None:
            ops.gemm(dy_full, x2, a_mn=True, b_mn=True, out=w_ref._tpb_grad_view,
                     accumulate=getattr(w_ref, "_tpb_grad_written", False))
            w_ref._tpb_grad_written = True
            dw = None
        else:
            dw = ops.gemm(dy_full, x2, a_mn=True, b_mn=True)
        return dx, dw, None, None


class TPContext:
    """Plans shared by the tensor-parallel linears of one model (keyed by shape)."""

    def __init__(self, group=None, arena_bytes: int = 4 << 30):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.cuda = torch.cuda.is_available()
        self.arena = None
        if self.cuda:
            self.arena = SymmArena._instance or SymmArena(arena_bytes, group=group)
        self._ag, self._rs, self._ar = {}, {}, {}

    def ar_plan(self, rows: int, hidden: int) -> "AllReduceNormPlan":
        key = (rows, hidden)
        if key not in self._ar:
            self._ar[key] = AllReduceNormPlan(self.arena, rows, hidden)
        return self._ar[key]

    def linear_allreduce_add_norm(self, a: torch.Tensor, weight: torch.Tensor, x: torch.Tensor,
                                  norm_w: Optional[torch.Tensor], eps: float) -> Optional[torch.Tensor]:
        """Row-parallel linear of a replicated small batch: ``x += sum_ranks(a @ weight.T)`` in place (``x`` is the
        replicated residual stream ``[rows, H]``) and returns ``rmsnorm(x) * norm_w`` (None without ``norm_w``).
        The GEMM writes its partial straight into the arena slice that the one-launch all-reduce reads."""
        if self.arena is not None and a.is_cuda and a.dtype == torch.bfloat16 and self.world > 1:
            plan = self.ar_plan(x.shape[0], x.shape[1])
            ops.gemm(a, weight, out=plan.partial()[: x.shape[0]])
            return plan.run(x, norm_w, eps)
        y = ops.linear(a, weight)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        x += y
        return None if norm_w is None else ops.rms_norm(x, norm_w, eps)

    def ag_plan(self, m_total: int, k: int) -> AGGemmPlan:
        key = (m_total, k)
        if key not in self._ag:
            rpf = 128 if (m_total // self.world) % 128 == 0 else (m_total // self.world)
            self._ag[key] = AGGemmPlan(self.arena, m_total, k, rows_per_flag=rpf)
        return self._ag[key]

    def rs_plan(self, m_total: int, n: int) -> GemmRSPlan:
        key = (m_total, n)
        if key not in self._rs:
            self._rs[key] = GemmRSPlan(self.arena, m_total, n)
        return self._rs[key]

    # ---- functional API
    def all_gather_linear(self, x_local: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``all_gather_rows(x_local) @ weight.T`` -> ``[rows * world, N_shard]``."""
        rows, k = x_local.reshape(-1, x_local.shape[-1]).shape
        m = rows * self.world
        if self.arena is not None and x_local.is_cuda and x_local.dtype == torch.bfloat16:
            return _AGLinearFn.apply(x_local, weight, self.ag_plan(m, k), self.rs_plan(m, k))
        return _ag_linear_ref(x_local.reshape(rows, k), weight, self.group)

    def linear_reduce_scatter(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``reduce_scatter_rows(x @ weight.T)`` -> ``[rows / world, N]``."""
        x2 = x.reshape(-1, x.shape[-1])
        m, n = x2.shape[0], weight.shape[0]
        if self.arena is not None and x.is_cuda and x.dtype == torch.bfloat16 and m % self.world == 0:
            return _LinearRSFn.apply(x2, weight, self.rs_plan(m, n), self.ag_plan(m, n))
        return _linear_rs_ref(x2, weight, self.group)


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = x.new_empty(x.shape[0] * w, *x.shape[1:])
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = g.new_empty(g.shape[0] // w, *g.shape[1:])
        _reduce_scatter(out, g.contiguous(), ctx.group)
        return out, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        w = dist.get_world_size(group)
        out = x.new_empty(x.shape[0] // w, *x.shape[1:])
        _reduce_scatter(out, x.contiguous(), group)
        return out

    @staticmethod
    def backward(ctx, g):
        w = dist.get_world_size(ctx.group)
        out = g.new_empty(g.shape[0] * w, *g.shape[1:])
        dist.all_gather_into_tensor(out, g.contiguous(), group=ctx.group)
        return out, None


def _reduce_scatter(out, inp, group):
    if dist.get_backend(group) == "gloo":
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp[r * out.shape[0]: (r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, inp, group=group)


def _ag_linear_ref(x_local, weight, group):
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return torch.nn.functional.linear(x_local, weight)
    return torch.nn.functional.linear(_AllGatherRows.apply(x_local, group), weight)


def _linear_rs_ref(x, weight, group):
    y = torch.nn.functional.linear(x, weight)
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return y
    return _ReduceScatterRows.apply(y, group)
