"""Context parallelism: ring attention over sequence shards.

Every rank holds one contiguous chunk of the sequence for q, k and v. Step ``s`` of the ring
attends the local queries to the K/V chunk of rank ``(rank - s) mod world``; the partial output is
folded into an fp32 accumulator by log-sum-exp. On CUDA the chunks live in the symmetric arena:
the next chunk is pulled from the peer's memory by a copy kernel on a side stream while the flash
kernel works on the current one, and the merge is one fused kernel (``csrc/kernels/cp_ops.cu``).
With ``causal`` a rank skips the chunks that lie entirely in its future, attends its own chunk
with the causal mask and earlier chunks without one. Backward walks the same ring with the global
LSE and returns the dK/dV partials to their owners with one reduce-scatter.

CPU tensors (gloo ranks) run the same schedule on plain PyTorch math, which is also the oracle.

Capability reference: tensorplay/distributed/tensor/experimental/_context_parallel/_attention.py
:243-408 (``_templated_ring_attention`` and its backward), :997-1086 (``context_parallel``,
``context_parallel_unshard``).
"""
from __future__ import annotations

import contextlib
import math
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _native
from ..ops._common import lib, stream_ptr
from ..ops.attention import flash_bwd, flash_fwd

_native._KERNEL_SIGS.setdefault(
    "tpb_attn_merge", [_native.P, _native.P, _native.P, _native.P, _native.I, _native.I, _native.I, _native.I,
                       _native.LL, _native.LL, _native.LL, _native.I, _native.I, _native.I, _native.P])


def _ref_attn_lse(q, k, v, causal: bool, scale: float):
    """fp32 attention returning (o [B, T, H, D] fp32, lse [B, H, T])."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(Tq, device=q.device).view(-1, 1)
        j = torch.arange(Tk, device=q.device).view(1, -1)
        s = s.masked_fill(j > i + (Tk - Tq), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    return torch.matmul(p, vf).permute(0, 2, 1, 3), lse, p


def merge_partials(acc: Optional[Tensor], lse_acc: Optional[Tensor], part: Tensor, lse_part: Tensor):
    """Fold ``(part, lse_part)`` into ``(acc fp32 [B, T, H, D], lse_acc [B, H, >=T])``; returns both."""
    B, T, H, D = part.shape
    first = acc is None
    if part.is_cuda:
        if first:
            acc = torch.empty(B, T, H, D, dtype=torch.float32, device=part.device)
            lse_acc = torch.empty_like(lse_part)
        k = lib()
        fn = k.tpb_attn_merge
        _native.check(fn(acc.data_ptr(), lse_acc.data_ptr(), part.data_ptr(), lse_part.data_ptr(), B, T, H, D,
                         part.stride(1), part.stride(2), part.stride(0), lse_acc.shape[2], lse_part.shape[2],
                         int(first), stream_ptr()), "tpb_attn_merge")
        return acc, lse_acc
    if first:
        return part.float().clone(), lse_part.clone()
    lse = torch.logaddexp(lse_acc, lse_part)
    wo = torch.exp(lse_acc - lse).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)
    wn = torch.exp(lse_part - lse).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)
    return acc * wo + part.float() * wn, lse


class _Ring:
    """K/V exchange of one ring pass: symmetric-memory pulls on CUDA, all-gather on CPU."""

    def __init__(self, k: Tensor, v: Tensor, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.k, self.v = k, v
        self.cuda = k.is_cuda
        if self.cuda:
            from .symm import SymmArena
            arena = SymmArena._instance
            if arena is None:
                raise RuntimeError("ring attention on CUDA needs the symmetric arena (create a SymmArena, "
                                   "an FSDPEngine with comm='symm', or a TPContext first)")
            self.arena = arena
            n = k.numel()
            key = ("cp_kv", n, k.dtype)
            cache = getattr(arena, "_cp_cache", None)
            if cache is None:
                cache = arena._cp_cache = {}
            if key not in cache:
                cache[key] = dict(buf=arena.alloc(2 * n, k.dtype), slot=arena.slots(self.world), epoch=0,
                                  stage=[torch.empty(2 * n, dtype=k.dtype, device=k.device) for _ in range(2)],
                                  stream=torch.cuda.Stream())
            st = self.st = cache[key]
            st["buf"][:n].copy_(k.reshape(-1))
            st["buf"][n:].copy_(v.reshape(-1))
            self._barrier()  # every rank's chunk is in place before anyone pulls
        else:
            ks = [torch.empty_like(k) for _ in range(self.world)]
            vs = [torch.empty_like(v) for _ in range(self.world)]
            dist.all_gather(ks, k.contiguous(), group=group)
            dist.all_gather(vs, v.contiguous(), group=group)
            self._all = list(zip(ks, vs))
        self._pending = {}

    def _barrier(self):
        from ..ops._common import status_word
        st = self.st
        st["epoch"] += 1
        _native.check(self.arena.raw.tpb_symm_barrier(self.arena.pad_off, st["slot"], st["epoch"], 30.0,
                                                      status_word(self.k.device).data_ptr(), stream_ptr()),
                      "tpb_symm_barrier")

    def prefetch(self, c: int, parity: int) -> None:
        """Start pulling chunk ``c`` into staging buffer ``parity`` on the side stream."""
        if not self.cuda or c == self.rank:
            return
        st = self.st
        side = st["stream"]
        side.wait_stream(torch.cuda.current_stream())
        dst = st["stage"][parity]
        with torch.cuda.stream(side):
            _native.check(self.arena.raw.tpb_symm_peer_copy(c, self.arena.offset_of(st["buf"]), dst.data_ptr(),
                                                            dst.numel() * dst.element_size(), 32,
                                                            side.cuda_stream), "tpb_symm_peer_copy")
            ev = torch.cuda.Event()
            ev.record(side)
        self._pending[c] = (parity, ev)

    def get(self, c: int):
        if c == self.rank:
            return self.k, self.v
        if not self.cuda:
            return self._all[c]
        parity, ev = self._pending.pop(c)
        torch.cuda.current_stream().wait_event(ev)
        n = self.k.numel()
        buf = self.st["stage"][parity]
        return buf[:n].view(self.k.shape), buf[n:].view(self.v.shape)

    def close(self):
        if self.cuda:
            self._barrier()  # peers are done reading this rank's chunk before it is overwritten


def _gids(rank: int, world: int, zigzag: bool) -> List[int]:
    """Global chunk ids of the parts a rank holds: one contiguous chunk, or (load-balanced for causal
    masks) chunk ``rank`` from the head and chunk ``2 * world - 1 - rank`` from the tail."""
    return [rank, 2 * world - 1 - rank] if zigzag else [rank]


def _plan(rank: int, world: int, causal: bool, zigzag: bool):
    """Ring order of the peers this rank needs and, per peer, the (q part, kv part, causal) pairs."""
    mine = _gids(rank, world, zigzag)
    steps = []
    for s in range(world):
        c = (rank - s) % world
        pairs = []
        for p, gi in enumerate(mine):
            for pp, gj in enumerate(_gids(c, world, zigzag)):
                if causal and gj > gi:
                    continue  # that chunk lies entirely in this part's future
                pairs.append((p, pp, causal and gi == gj))
        if pairs:
            steps.append((c, pairs))
    return steps


class _RingAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, group, zigzag):
        ring = _Ring(k, v, group)
        rank, world = ring.rank, ring.world
        steps = _plan(rank, world, causal, zigzag)
        P = 2 if zigzag else 1
        Tc = q.shape[1] // P
        acc, lse = [None] * P, [None] * P
        if len(steps) > 1:
            ring.prefetch(steps[1][0], 1)
        for i, (c, pairs) in enumerate(steps):
            kc, vc = ring.get(c)
            for p, pp, cz in pairs:
                qp = q[:, p * Tc: (p + 1) * Tc]
                kp, vp = kc[:, pp * Tc: (pp + 1) * Tc], vc[:, pp * Tc: (pp + 1) * Tc]
                if q.is_cuda:
                    o_s, lse_s = flash_fwd(qp, kp, vp, cz, scale)
                else:
                    o_s, lse_s, _ = _ref_attn_lse(qp, kp, vp, cz, scale)
                acc[p], lse[p] = merge_partials(acc[p], lse[p], o_s, lse_s)
            # staging buffer i & 1 is free once the kernels just enqueued have read it: the pull of
            # the next-but-one peer is ordered after them and overlaps with the next step's attention
            if i + 2 < len(steps):
                ring.prefetch(steps[i + 2][0], i & 1)
        ring.close()
        out = torch.cat([a.to(q.dtype) for a in acc], dim=1)
        ctx.save_for_backward(q, k, v, out, *lse)
        ctx.causal, ctx.scale, ctx.group, ctx.zigzag = causal, scale, group, zigzag
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out = ctx.saved_tensors[:4]
        lse = ctx.saved_tensors[4:]
        causal, scale, group, zigzag = ctx.causal, ctx.scale, ctx.group, ctx.zigzag
        ring = _Ring(k, v, group)
        rank, world = ring.rank, ring.world
        steps = _plan(rank, world, causal, zigzag)
        P = 2 if zigzag else 1
        Tc = q.shape[1] // P
        do = do.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        dkv = torch.zeros((world, 2) + tuple(k.shape), dtype=torch.float32, device=k.device)
        if len(steps) > 1:
            ring.prefetch(steps[1][0], 1)
        for i, (c, pairs) in enumerate(steps):
            kc, vc = ring.get(c)
            for p, pp, cz in pairs:
                sl, sk = slice(p * Tc, (p + 1) * Tc), slice(pp * Tc, (pp + 1) * Tc)
                args = (do[:, sl], q[:, sl], kc[:, sk], vc[:, sk], out[:, sl], lse[p], cz, scale)
                dq_s, dk_s, dv_s = flash_bwd(*args) if q.is_cuda else _ref_bwd(*args)
                dq[:, sl] += dq_s.float()
                dkv[c, 0, :, sk] += dk_s.float()
                dkv[c, 1, :, sk] += dv_s.float()
            if i + 2 < len(steps):
                ring.prefetch(steps[i + 2][0], i & 1)
        ring.close()
        # partials for the chunks of rank c go back to rank c, summed over the ranks that attended them
        mine = torch.empty((2,) + tuple(k.shape), dtype=torch.float32, device=k.device)
        if k.is_cuda:
            dist.reduce_scatter_tensor(mine, dkv, group=group)
        else:
            dist.all_reduce(dkv, group=group)
            mine = dkv[rank]
        return dq.to(q.dtype), mine[0].to(k.dtype), mine[1].to(v.dtype), None, None, None, None


def _ref_bwd(do, q, k, v, out, lse, causal, scale):
    """fp32 backward of one ring step given the global LSE (``lse`` [B, H, T])."""
    B, Tq, Hq, D = q.shape
    Tk, Hkv = k.shape[1], k.shape[2]
    g = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    dof = do.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        i = torch.arange(Tq, device=q.device).view(-1, 1)
        j = torch.arange(Tk, device=q.device).view(1, -1)
        s = s.masked_fill(j > i + (Tk - Tq), float("-inf"))
    p = torch.exp(s - lse[:, :, :Tq].unsqueeze(-1))
    delta = (out.float() * do.float()).sum(-1).permute(0, 2, 1).unsqueeze(-1)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf).permute(0, 2, 1, 3)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    dk = dk.view(B, Hkv, g, Tk, D).sum(2).permute(0, 2, 1, 3)
    dv = dv.view(B, Hkv, g, Tk, D).sum(2).permute(0, 2, 1, 3)
    return dq, dk, dv


def ring_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool = True, scale: Optional[float] = None,
                   group=None, load_balance: bool = False) -> Tensor:
    """Attention over a sequence sharded across ``group``; inputs and output are this rank's share,
    ``[B, T_local, H, D]``. ``load_balance=False``: rank r holds the r-th contiguous chunk.
    ``load_balance=True`` (for causal masks): the sequence is cut into ``2 * world`` chunks and rank r
    holds chunks ``r`` and ``2 * world - 1 - r`` (see :func:`context_parallel_shard`), so that every
    rank attends the same number of chunk pairs."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        from ..ops.attention import flash_attention
        return flash_attention(q, k, v, causal, scale)
    if load_balance and q.shape[1] % 2:
        raise ValueError("load-balanced context parallelism needs an even local sequence length")
    return _RingAttnFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), causal, scale, group, bool(load_balance))


# ---------------------------------------------------------------------------- sharding helpers
def context_parallel_shard(buffers: Sequence[Tensor], seq_dims: Sequence[int], group=None,
                           load_balance: bool = False) -> List[Tensor]:
    """This rank's share of every buffer along its sequence dim: the rank-th contiguous chunk, or with
    ``load_balance`` the head chunk ``rank`` and the tail chunk ``2 * world - 1 - rank`` of ``2 * world``
    chunks, concatenated (tensorplay/distributed/tensor/experimental/_context_parallel/_load_balancer.py:26-47)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    n = 2 * world if load_balance else world
    out = []
    for b, d in zip(buffers, seq_dims):
        if b.shape[d] % n:
            raise ValueError(f"sequence length {b.shape[d]} is not divisible by {n}")
        ch = b.chunk(n, dim=d)
        out.append(torch.cat((ch[rank], ch[n - 1 - rank]), dim=d).contiguous() if load_balance else ch[rank].contiguous())
    return out


def context_parallel_unshard(buffers: Sequence[Tensor], seq_dims: Sequence[int], group=None,
                             load_balance: bool = False) -> List[Tensor]:
    """All-gather the shares back into full sequences (undoing the head-tail interleave if used)."""
    world = dist.get_world_size(group)
    out = []
    for b, d in zip(buffers, seq_dims):
        parts = [torch.empty_like(b) for _ in range(world)]
        dist.all_gather(parts, b.contiguous(), group=group)
        if load_balance:
            halves = [p.chunk(2, dim=d) for p in parts]
            parts = [h[0] for h in halves] + [h[1] for h in reversed(halves)]
        out.append(torch.cat(parts, dim=d))
    return out


_cp_group = None


@contextlib.contextmanager
def context_parallel(group=None, buffers: Sequence[Tensor] = (), buffer_seq_dims: Sequence[int] = ()):
    """Inside the context ``nn.GroupedQueryAttention`` / ``ops.flash_attention`` users that call
    :func:`current_group` route attention through :func:`ring_attention`; ``buffers`` are sharded in
    place along their sequence dims for the duration."""
    global _cp_group
    saved = [b.clone() for b in buffers]
    for b, d, s in zip(buffers, buffer_seq_dims, context_parallel_shard(buffers, buffer_seq_dims, group)):
        b.resize_(s.shape).copy_(s)
    prev, _cp_group = _cp_group, (group if group is not None else dist.group.WORLD)
    try:
        yield
    finally:
        _cp_group = prev
        for b, s in zip(buffers, saved):
            b.resize_(s.shape).copy_(s)


def current_group():
    """The context-parallel group set by :func:`context_parallel`, or ``None``."""
    return _cp_group
