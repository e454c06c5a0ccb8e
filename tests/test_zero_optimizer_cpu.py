"""ZeRO-1 optimizer on gloo ranks: same trajectory as the unsharded optimizer, state sharded, state dict
consolidated and reloaded, uneven inputs through Join."""
import torch

from tensorplay_b200.distributed.algorithms.join import Join

from tests.distutil import run_ranks


def _net():
    from torch import nn
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(12, 24), nn.Tanh(), nn.Linear(24, 7), nn.Tanh(), nn.Linear(7, 3))


def _worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer as ZeRO

    ref, net = _net(), _net()
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.1)
    zopt = ZeRO(net.parameters(), torch.optim.AdamW, lr=1e-2, weight_decay=0.1)
    owned = [p for g in zopt.optim.param_groups for p in g["params"]]
    assert 0 < len(owned) < len(list(net.parameters()))

    def run(model, opt, steps, lr=None):
        for s in range(steps):
            g = torch.Generator().manual_seed(s)
            x = torch.randn(world, 4, 12, generator=g)
            # the same (already averaged) gradient on every rank, as after DDP's reduction
            model.zero_grad()
            sum(model(x[r]).square().mean() for r in range(world)).div(world).backward()
            if lr is not None:
                for grp in opt.param_groups:
                    grp["lr"] = lr
            opt.step()

    run(ref, ropt, 3); run(net, zopt, 3)
    for a, b in zip(ref.parameters(), net.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)
    # a scheduler-style change of lr on the outer groups reaches the local optimizer
    run(ref, ropt, 2, lr=5e-3); run(net, zopt, 2, lr=5e-3)
    for a, b in zip(ref.parameters(), net.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)
    # sharded: state only for the owned parameters
    assert len(zopt.optim.state) == len(owned)

    # consolidate on rank 1, compare with the unsharded optimizer's state dict, ship it to everyone, reload
    zopt.consolidate_state_dict(to=1)
    box = [None]
    if rank == 1:
        sd = zopt.state_dict()
        rsd = ropt.state_dict()
        assert sorted(sd["state"]) == sorted(rsd["state"])
        for i in sd["state"]:
            torch.testing.assert_close(sd["state"][i]["exp_avg"], rsd["state"][i]["exp_avg"], rtol=1e-6, atol=1e-8)
        assert [g["params"] for g in sd["param_groups"]] == [g["params"] for g in rsd["param_groups"]]
        box[0] = sd
    else:
        import pytest
        with pytest.raises(RuntimeError):
            zopt.state_dict()
    dist.broadcast_object_list(box, src=1)
    net2 = _net()
    net2.load_state_dict(net.state_dict())
    z2 = ZeRO(net2.parameters(), torch.optim.AdamW, lr=1e-2, weight_decay=0.1)
    z2.load_state_dict(box[0])
    run(ref, ropt, 2); run(net2, z2, 2)
    for a, b in zip(ref.parameters(), net2.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-6, atol=1e-7)

    # parameter groups with their own hyper-parameters, and a group added later
    from torch import nn
    torch.manual_seed(1)
    a, b = nn.Linear(4, 4), nn.Linear(4, 4)
    a2, b2 = nn.Linear(4, 4), nn.Linear(4, 4)
    a2.load_state_dict(a.state_dict()); b2.load_state_dict(b.state_dict())
    r = torch.optim.SGD([{"params": a.parameters(), "lr": 0.1}], lr=0.01, momentum=0.9)
    z = ZeRO([{"params": list(a2.parameters()), "lr": 0.1}], torch.optim.SGD, lr=0.01, momentum=0.9)
    r.add_param_group({"params": list(b.parameters())})
    z.add_param_group({"params": list(b2.parameters())})
    for s in range(3):
        x = torch.randn(5, 4, generator=torch.Generator().manual_seed(s))
        for m1, m2, o in ((a, b, r), (a2, b2, z)):
            o.zero_grad()
            m2(m1(x)).sum().backward()
            o.step()
    for p, q in zip(list(a.parameters()) + list(b.parameters()), list(a2.parameters()) + list(b2.parameters())):
        torch.testing.assert_close(p, q, rtol=1e-6, atol=1e-7)
    return True


def test_zero_matches_unsharded_optimizer():
    assert all(run_ranks(_worker, 2))


def _join_worker(rank, world):
    from tensorplay_b200.distributed.algorithms.join import Join
    from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer as ZeRO

    net = _net()
    z = ZeRO(net.parameters(), torch.optim.SGD, lr=0.1)
    steps = 2 + rank          # uneven: rank 1 takes one more step than rank 0
    with Join([z]):
        for s in range(steps):
            net.zero_grad()
            net(torch.ones(2, 12) * (s + 1)).sum().backward()
            z.step()
    # both ranks hold the same parameters after the join
    import torch.distributed as dist
    flat = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
    got = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(got, flat)
    torch.testing.assert_close(got[0], got[1])
    return True


def test_zero_with_uneven_inputs():
    assert all(run_ranks(_join_worker, 2))


def _ddp_join_worker(rank, world):
    import torch.distributed as dist
    from torch import nn
    from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP
    from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer as ZeRO

    net = _net()
    ddp = DDP(net, bucket_cap_mb=0.001)
    opt = ZeRO(net.parameters(), torch.optim.SGD, lr=0.05)
    steps = 2 + 2 * rank      # rank 1 trains two iterations longer
    with Join([ddp, opt]):
        for s in range(steps):
            net.zero_grad(set_to_none=False)
            ddp(torch.ones(2, 12) * (s + 1 + rank)).sum().backward()
            opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in net.parameters()])
    got = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(got, flat)
    torch.testing.assert_close(got[0], got[1])

    # oracle: the same schedule on one process, absent ranks contributing zero gradients
    ref = _net()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
    for s in range(2 + 2 * (world - 1)):
        ref.zero_grad()
        live = [r for r in range(world) if s < 2 + 2 * r]
        (sum(ref(torch.ones(2, 12) * (s + 1 + r)).sum() for r in live) / world).backward()
        ropt.step()
    for a, b in zip(ref.parameters(), net.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)

    # early termination raises on every rank instead of shadowing
    import pytest
    ddp2 = DDP(_net(), bucket_cap_mb=0.001)
    with pytest.raises(RuntimeError, match="exhausted"):
        with ddp2.join(throw_on_early_termination=True):
            for s in range(1 + rank):
                ddp2(torch.ones(2, 12)).sum().backward()
    return True


def test_ddp_and_zero_join_with_uneven_inputs():
    assert all(run_ranks(_ddp_join_worker, 2))
