"""Model averaging, the 8-bit quantisation hooks and the post-local-SGD hook on gloo ranks."""
from collections import OrderedDict

import torch

from tests.distutil import run_ranks


def _avg_worker(rank, world):
    import torch.distributed as dist
    from torch import nn
    from tensorplay_b200.distributed.algorithms import model_averaging as MA

    torch.manual_seed(0)
    net = nn.Linear(5, 3)
    half = nn.Linear(3, 2).to(torch.bfloat16)
    params = list(net.parameters()) + list(half.parameters())
    for p in params:
        p.data.fill_(float(rank + 1))
        p.grad = torch.zeros_like(p)
    MA.average_parameters(params)
    mean = sum(range(1, world + 1)) / world
    assert all(torch.allclose(p.float(), torch.full_like(p, mean, dtype=torch.float32)) for p in params)

    # periodic: warm-up of 2 steps, then every 3rd step
    av = MA.PeriodicModelAverager(period=3, warmup_steps=2)
    averaged_at = []
    for step in range(9):
        for p in params:
            p.data.fill_(float(rank))
        av.average_parameters(params)
        if torch.allclose(params[0], torch.full_like(params[0], (world - 1) / 2)) and world > 1:
            averaged_at.append(step)
    assert averaged_at == [2, 5, 8], averaged_at

    # parameter groups as an optimizer holds them; parameters without gradient stay
    net2 = nn.Linear(2, 2)
    net2.weight.data.fill_(float(rank)); net2.bias.data.fill_(float(rank))
    net2.weight.grad = torch.zeros_like(net2.weight)
    opt = torch.optim.SGD(net2.parameters(), lr=0.1)
    MA.PeriodicModelAverager(period=1).average_parameters(opt.param_groups)
    assert torch.allclose(net2.weight, torch.full_like(net2.weight, (world - 1) / 2))
    assert torch.allclose(net2.bias, torch.full_like(net2.bias, float(rank)))
    return True


def test_periodic_model_averager():
    assert all(run_ranks(_avg_worker, 2))


def _hier_worker(rank, world):
    import pytest
    from torch import nn
    from tensorplay_b200.distributed.algorithms.model_averaging import HierarchicalModelAverager

    with pytest.raises(ValueError):
        HierarchicalModelAverager(OrderedDict([(2, 2), (4, 3)]))
    av = HierarchicalModelAverager(OrderedDict([(2, 2), (4, world)]), warmup_steps=1)
    p = nn.Parameter(torch.zeros(3))
    p.grad = torch.zeros(3)
    seen = []
    for step in range(9):
        p.data.fill_(float(rank))
        av.average_parameters([p])
        seen.append(round(p.data[0].item(), 3))
    pair = (rank // 2) * 2 + 0.5           # mean of ranks {0,1} or {2,3}
    glob = (world - 1) / 2
    want = [float(rank)] * 9
    for step in range(1, 9):
        if step % 4 == 0:
            want[step] = glob
        elif step % 2 == 0:
            want[step] = pair
    assert seen == want, (rank, seen, want)
    return True


def test_hierarchical_model_averager():
    assert all(run_ranks(_hier_worker, 4))


def _hooks_worker(rank, world):
    import torch.distributed as dist
    from torch import nn
    from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP
    from tensorplay_b200.distributed.algorithms import ddp_comm_hooks as H

    def grads(hook, state, steps=1):
        torch.manual_seed(0)
        net = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 4))
        ddp = DDP(net, bucket_cap_mb=0.001)
        if hook is not None:
            ddp.register_comm_hook(state, hook)
        out = None
        for s in range(steps):
            net.zero_grad(set_to_none=False)
            g = torch.Generator().manual_seed(10 * s + rank)
            ddp(torch.randn(8, 16, generator=g)).square().mean().backward()
            out = torch.cat([p.grad.reshape(-1).clone() for p in net.parameters()])
        return out

    ref = grads(None, None)
    for hook, kw in ((H.quantization_hooks.quantization_pertensor_hook, {}),
                     (H.quantization_hooks.quantization_perchannel_hook, {})):
        got = grads(hook, None)
        # 8 bits over the bucket's range: error below one quantisation step of the widest bucket
        assert (got - ref).abs().max() <= ref.abs().max() * 2 / 255 + 1e-7, (got - ref).abs().max()

    local = grads(H.noop_hook, None)
    assert not torch.allclose(local, ref)

    # post-local SGD: all-reduced for two iterations, then local (no subgroup)
    st = H.PostLocalSGDState(None, None, start_localSGD_iter=2)
    a = grads(H.post_localSGD.post_localSGD_hook, st, steps=2)
    assert st.iter == 2
    st2 = H.PostLocalSGDState(None, None, start_localSGD_iter=2)
    b = grads(H.post_localSGD.post_localSGD_hook, st2, steps=3)
    gathered = [torch.empty_like(a) for _ in range(world)]
    dist.all_gather(gathered, a)
    assert all(torch.allclose(g, gathered[0]) for g in gathered)          # still synchronised
    dist.all_gather(gathered, b)
    assert not torch.allclose(gathered[0], gathered[1])                   # third iteration is local
    return True


def test_quantization_and_local_sgd_hooks():
    assert all(run_ranks(_hooks_worker, 2))
