"""DDP communication hooks and ``Join`` (tensorplay/distributed/algorithms/ddp_comm_hooks/*.py,
algorithms/join.py). Hooks follow the contract ``hook(state, bucket) -> Future[Tensor]``."""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.algorithms import Join, Joinable, JoinHook  # noqa: F401


def _done(t):
    f = torch.futures.Future()
    f.set_result(t)
    return f


def allreduce_hook(process_group, bucket):
    t = bucket.buffer()
    w = dist.get_world_size(process_group)
    dist.all_reduce(t, group=process_group)
    return _done(t.div_(w))


def _compress_hook(dtype):
    def hook(process_group, bucket):
        t = bucket.buffer()
        w = dist.get_world_size(process_group)
        c = t.to(dtype).div_(w)
        dist.all_reduce(c, group=process_group)
        return _done(t.copy_(c))
    return hook


fp16_compress_hook = _compress_hook(torch.float16)
bf16_compress_hook = _compress_hook(torch.bfloat16)


def powerSGD_hook(state, bucket):
    """Rank-``r`` PowerSGD with error feedback (one power iteration per step)."""
    t = bucket.buffer()
    n = t.numel()
    pg, r = state.get("process_group"), state.get("rank", 1)
    w = dist.get_world_size(pg)
    side = int(n ** 0.5)
    if side < 2 * r:
        dist.all_reduce(t, group=pg)
        return _done(t.div_(w))
    m = t[: side * side].view(side, side)
    err = state.setdefault("err", {}).setdefault(bucket.index(), torch.zeros_like(m))
    m.add_(err)
    if bucket.index() not in state.setdefault("q", {}):
        # the same start matrix on every rank (P = sum_r M_r Q needs one Q): seeded, not the global RNG
        g = torch.Generator().manual_seed(state.get("seed", 0) + bucket.index())
        state["q"][bucket.index()] = torch.randn(side, r, generator=g).to(device=t.device, dtype=t.dtype)
    q = state["q"][bucket.index()]
    p = m @ q
    dist.all_reduce(p, group=pg)
    p, _ = torch.linalg.qr(p.float())
    p = p.to(t.dtype)
    q = m.t() @ p
    dist.all_reduce(q, group=pg)
    q.div_(w)
    approx = p @ q.t()
    err.copy_(m - approx)
    m.copy_(approx)
    state["q"][bucket.index()] = q
    tail = t[side * side:]
    if tail.numel():
        dist.all_reduce(tail, group=pg)
        tail.div_(w)
    return _done(t)
