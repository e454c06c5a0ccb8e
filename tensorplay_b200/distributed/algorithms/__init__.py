"""DDP communication hooks and ``Join`` (tensorplay/distributed/algorithms/ddp_comm_hooks/*.py,
algorithms/join.py). Hooks follow the contract ``hook(state, bucket) -> Future[Tensor]``."""
from __future__ import annotations

import torch
import torch.distributed as dist
from .join import Join, Joinable, JoinHook  # noqa: F401


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


# ---------------------------------------------------------------- quantisation and local-SGD hooks
def _quantize_per_tensor(x: torch.Tensor):
    lo, hi = x.min(), x.max()
    scale = ((hi - lo) / 255.0).clamp_min(1e-12)
    q = ((x - lo) / scale).round_().clamp_(0, 255).to(torch.uint8)
    return q, scale.reshape(1), lo.reshape(1)


def quantization_pertensor_hook(process_group, bucket):
    """All-gather of the bucket quantised to 8 bits with one (scale, zero point) per rank, de-quantised and
    averaged locally: a quarter of the bytes of an fp32 all-reduce on the wire
    (tensorplay/distributed/algorithms/ddp_comm_hooks/quantization_hooks.py)."""
    t = bucket.buffer()
    pg = process_group if process_group is not None else dist.group.WORLD
    w = dist.get_world_size(pg)
    q, scale, lo = _quantize_per_tensor(t.float())
    qs = [torch.empty_like(q) for _ in range(w)]
    meta = torch.cat((scale, lo))
    metas = [torch.empty_like(meta) for _ in range(w)]
    dist.all_gather(qs, q, group=pg)
    dist.all_gather(metas, meta, group=pg)
    acc = torch.zeros_like(t, dtype=torch.float32)
    for qi, mi in zip(qs, metas):
        acc += qi.float() * mi[0] + mi[1]
    return _done(t.copy_((acc / w).to(t.dtype)))


def quantization_perchannel_hook(process_group, bucket, bucket_size: int = 512):
    """Like the per-tensor hook with one (scale, zero point) per ``bucket_size`` consecutive elements."""
    t = bucket.buffer()
    pg = process_group if process_group is not None else dist.group.WORLD
    w = dist.get_world_size(pg)
    n = t.numel()
    pad = (-n) % bucket_size
    x = torch.nn.functional.pad(t.float(), (0, pad)).view(-1, bucket_size)
    lo, hi = x.min(dim=1, keepdim=True).values, x.max(dim=1, keepdim=True).values
    scale = ((hi - lo) / 255.0).clamp_min(1e-12)
    q = ((x - lo) / scale).round_().clamp_(0, 255).to(torch.uint8)
    meta = torch.cat((scale, lo), dim=1)
    qs = [torch.empty_like(q) for _ in range(w)]
    metas = [torch.empty_like(meta) for _ in range(w)]
    dist.all_gather(qs, q, group=pg)
    dist.all_gather(metas, meta, group=pg)
    acc = torch.zeros_like(x)
    for qi, mi in zip(qs, metas):
        acc += qi.float() * mi[:, :1] + mi[:, 1:]
    return _done(t.copy_((acc / w).view(-1)[:n].to(t.dtype)))


class PostLocalSGDState:
    """State of :func:`post_localSGD_hook`: gradients are all-reduced over ``process_group`` for the first
    ``start_localSGD_iter`` iterations, afterwards only over ``subgroup`` (``None``: not at all), and the model
    is averaged globally by a ``PeriodicModelAverager`` (post_localSGD_hook.py in the reference)."""

    def __init__(self, process_group, subgroup, start_localSGD_iter: int, post_local_gradient_allreduce: bool = True):
        self.process_group, self.subgroup = process_group, subgroup
        self.start_localSGD_iter = start_localSGD_iter
        self.post_local_gradient_allreduce = post_local_gradient_allreduce
        self.iter = 0

    def maybe_increase_iter(self, bucket) -> None:
        if bucket.is_last():
            self.iter += 1


def post_localSGD_hook(state: PostLocalSGDState, bucket):
    t = bucket.buffer()
    if state.iter < state.start_localSGD_iter:
        state.maybe_increase_iter(bucket)
        return allreduce_hook(state.process_group, bucket)
    state.maybe_increase_iter(bucket)
    if not state.post_local_gradient_allreduce or state.subgroup is None:
        return _done(t)
    return allreduce_hook(state.subgroup, bucket)
