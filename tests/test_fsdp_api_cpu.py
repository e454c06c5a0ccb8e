"""The public ``fully_shard`` / ``FullyShardedDataParallel`` API on gloo ranks: one collective per
unit, hybrid sharding on a 2-D mesh, custom communication objects, the all-reduce hook, CPU
offload, gradient accumulation without synchronisation, the FSDP1 facade's helpers, and loud
failures for arguments that are not implemented (restated from the reference's
test/distributed/test_fsdp_e2e.py:202-498)."""
import copy

import pytest
import torch
from torch import nn

from tests.distutil import run_ranks


def _net(seed=0):
    torch.manual_seed(seed)
    # row counts that do not divide by the world sizes used below, a bias-free layer and a 0-dim parameter
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(12, 7)
            self.b = nn.Sequential(nn.Linear(7, 10), nn.Tanh(), nn.Linear(10, 5, bias=False))
            self.scale = nn.Parameter(torch.tensor(1.5))

        def forward(self, x):
            return self.b(torch.tanh(self.a(x))) * self.scale

    return Net()


def _dense_grads(seed, xs):
    m = _net(seed)
    for x in xs:
        m(x).pow(2).mean().backward()
    return {n: p.grad.clone() / len(xs) for n, p in m.named_parameters()}, m


def _full_grad(state, info):
    """Gather a sharded gradient back to the full tensor."""
    import torch.distributed as dist
    g = info.sharded.grad
    pad = torch.zeros((info.chunk,) + info.rest, dtype=g.dtype)
    pad[: info.local_rows] = g
    out = [torch.zeros_like(pad) for _ in range(state.world)]
    dist.all_gather(out, pad, group=state.group)
    return torch.cat(out)[: info.n0].reshape(info.full_shape)


def _hsdp_worker(rank, world):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from tensorplay_b200.distributed.fsdp import fully_shard
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("replicate", "shard"))
    m = _net(3)
    fully_shard(m.b, mesh=mesh)
    fully_shard(m, mesh=mesh)
    torch.manual_seed(100)
    xs = [torch.randn(4, 12) for _ in range(world)]
    m(xs[rank]).pow(2).mean().backward()
    ref, _ = _dense_grads(3, xs)
    worst = 0.0
    for st in m._fsdp_state.tree(True):
        assert st.collective_counts == {"all_gather": 1, "reduce_scatter": 1, "all_reduce": 1}, st.collective_counts
        assert st.world == 2 and st.rep_world == 2
        for info in st.params:
            worst = max(worst, float((_full_grad(st, info) - ref[_name_of(m, info)]).abs().max()))
    # all-reduce switched off: the reduce-scattered partial sums wait, then one all-reduce delivers both
    m.zero_grad(set_to_none=True)
    m.set_requires_all_reduce(False)
    m(xs[rank]).pow(2).mean().backward()
    assert all(st.partial is not None for st in m._fsdp_state.tree(True))
    m.set_requires_all_reduce(True)
    m(xs[rank]).pow(2).mean().backward()
    for st in m._fsdp_state.tree(True):
        for info in st.params:
            worst = max(worst, float((_full_grad(st, info) - 2 * ref[_name_of(m, info)]).abs().max()))
    return worst


def _name_of(root, info):
    for n, mod in root.named_modules():
        if mod is info.module:
            return (n + "." if n else "") + info.name
    raise KeyError(info.name)


def test_hybrid_sharding_on_a_2d_mesh_reduces_over_both_dimensions():
    for worst in run_ranks(_hsdp_worker, 4):
        assert worst < 1e-6, worst


def _knobs_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.fsdp import (AllGather, CPUOffloadPolicy, MixedPrecisionPolicy, ReduceScatter,
                                                  fully_shard, register_fsdp_forward_method)
    calls = {"ag": 0, "rs": 0, "alloc": 0, "hook": 0}

    class MyAG(AllGather):
        def allocate(self, size, *, dtype, device):
            calls["alloc"] += 1
            return torch.empty(tuple(size), dtype=dtype, device=device)

        def __call__(self, output_tensor, input_tensor, group, async_op=False):
            calls["ag"] += 1
            return dist.all_gather_into_tensor(output_tensor, input_tensor, group=group)

    class MyRS(ReduceScatter):
        def allocate(self, size, *, dtype, device):
            calls["alloc"] += 1
            return torch.empty(tuple(size), dtype=dtype, device=device)

        def __call__(self, output_tensor, input_tensor, group, op, async_op=False):
            calls["rs"] += 1
            dist.all_reduce(input_tensor, op=op, group=group)
            n = output_tensor.numel()
            output_tensor.copy_(input_tensor.view(-1)[dist.get_rank(group) * n: (dist.get_rank(group) + 1) * n])

    torch.manual_seed(100)
    xs = [torch.randn(4, 12) for _ in range(world)]
    ref, dense = _dense_grads(5, xs)
    m = _net(5)
    fully_shard(m, offload_policy=CPUOffloadPolicy(pin_memory=False),
                mp_policy=MixedPrecisionPolicy(reduce_dtype=torch.float64))
    m.set_custom_all_gather(MyAG())
    m.set_custom_reduce_scatter(MyRS())
    m.set_all_reduce_hook(lambda t: calls.__setitem__("hook", calls["hook"] + 1))
    # accumulation without synchronisation, then a synchronised backward: one reduction for both
    m.set_requires_gradient_sync(False)
    m(xs[rank]).pow(2).mean().backward()
    assert calls["rs"] == 0 and all(p.grad is None for p in m.parameters())
    m.set_requires_gradient_sync(True)
    m(xs[rank]).pow(2).mean().backward()
    assert calls == {"ag": 2, "rs": 1, "alloc": 3, "hook": 1}, calls
    st = m._fsdp_state
    worst = max(float((_full_grad(st, i) - 2 * ref[_name_of(m, i)]).abs().max()) for i in st.params)
    assert st.flat_shard.device.type == "cpu" and st.flat_grad.device.type == "cpu"
    # sharded parameters are views of the flat shard: an optimizer step moves the gathered weights
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    opt.step()
    m.unshard()
    w = m.a.weight.detach().clone()
    m.reshard()
    want = dense.a.weight.detach() - 0.1 * 2 * ref["a.weight"]
    worst = max(worst, float((w - want).abs().max()))
    # a method other than forward can be made to gather / free like forward
    m2 = _net(5)
    m2.double_forward = lambda x: m2.forward(x) * 2
    fully_shard(m2)
    register_fsdp_forward_method(m2, "double_forward")
    y = m2.double_forward(xs[rank])
    assert torch.allclose(y, 2 * dense(xs[rank]), atol=1e-6)
    return worst


def test_custom_comm_hook_offload_accumulation_and_forward_method():
    for worst in run_ranks(_knobs_worker, 2):
        assert worst < 1e-6, worst


def _facade_worker(rank, world):
    from tensorplay_b200.distributed.fsdp import FullyShardedDataParallel as FSDP
    dense = _net(9)
    f = FSDP(_net(9), auto_wrap_policy=lambda mod, recurse, n: isinstance(mod, nn.Sequential))
    full = f.full_state_dict()
    for n, p in dense.named_parameters():
        assert torch.equal(full[n], p.detach()), n
    with f.summon_full_params(writeback=True):
        f.module.a.weight.data.mul_(2.0)
    assert torch.equal(f.full_state_dict()["a.weight"], 2 * dense.a.weight.detach())
    torch.manual_seed(100)
    xs = [torch.randn(4, 12) for _ in range(world)]
    f(xs[rank]).pow(2).mean().backward()
    dense.a.weight.data.mul_(2.0)
    for x in xs:
        (dense(x).pow(2).mean() / world).backward()
    want = torch.nn.utils.clip_grad_norm_(dense.parameters(), 0.01)
    got = f.clip_grad_norm_(0.01)
    return abs(float(got) - float(want))


def test_fsdp1_facade_state_dict_writeback_and_global_clip():
    for err in run_ranks(_facade_worker, 2):
        assert err < 1e-6, err


def test_unimplemented_arguments_raise():
    from tensorplay_b200.distributed.fsdp import FullyShardedDataParallel, ShardingStrategy, fully_shard
    with pytest.raises(NotImplementedError):
        fully_shard(_net(), shard_placement_fn=lambda p: None)
    with pytest.raises(NotImplementedError):
        fully_shard(_net(), reshard_after_forward=2)
    with pytest.raises(NotImplementedError):
        FullyShardedDataParallel(_net(), use_orig_params=False)
    with pytest.raises(NotImplementedError):
        FullyShardedDataParallel(_net(), sharding_strategy=ShardingStrategy.NO_SHARD)
    m = fully_shard(_net())
    with pytest.raises(ValueError):
        fully_shard(m)
    with pytest.raises(NotImplementedError):
        m.set_symm_mem_for_comm()
    # world size 1: a step through the hooks equals the dense step
    dense = _net()
    x = torch.randn(3, 12)
    m(x).sum().backward()
    dense(x).sum().backward()
    for (n, p), (_, q) in zip(m.named_parameters(), dense.named_parameters()):
        assert torch.allclose(p.grad.reshape(q.grad.shape), q.grad, atol=1e-6), n


def _state_dict_types_worker(rank, world):
    """Model and optimizer state in the FULL and SHARDED forms: a second model + optimizer loaded from either
    continues training exactly like the first."""
    from tensorplay_b200.distributed.fsdp import (FullOptimStateDictConfig, FullStateDictConfig, ShardedGradScaler,
                                                  StateDictType)
    from tensorplay_b200.distributed.fsdp import FullyShardedDataParallel as FSDP
    wrap = dict(auto_wrap_policy=lambda mod, recurse, n: isinstance(mod, nn.Sequential))
    f = FSDP(_net(3), **wrap)
    opt = torch.optim.AdamW(f.parameters(), lr=1e-2)
    torch.manual_seed(50 + rank)
    for _ in range(2):
        opt.zero_grad()
        f(torch.randn(4, 12)).pow(2).mean().backward()
        opt.step()
    assert FSDP.get_state_dict_type(f).state_dict_type == StateDictType.FULL_STATE_DICT
    full_sd = f.state_dict()
    dense = _net(3)
    assert set(full_sd) == set(dense.state_dict()) and full_sd["a.weight"].shape == dense.a.weight.shape
    full_osd = FSDP.optim_state_dict(f, opt)
    assert full_osd["state"]["a.weight"]["exp_avg"].shape == dense.a.weight.shape
    with FSDP.state_dict_type(f, StateDictType.FULL_STATE_DICT, FullStateDictConfig(rank0_only=True, offload_to_cpu=True),
                              FullOptimStateDictConfig(rank0_only=True)):
        r0 = f.state_dict()
        r0o = FSDP.optim_state_dict(f, opt)
    assert (len(r0) > 0) == (rank == 0) and (len(r0o) > 0) == (rank == 0)
    with FSDP.state_dict_type(f, StateDictType.SHARDED_STATE_DICT):
        sh_sd = f.state_dict()
        sh_osd = FSDP.optim_state_dict(f, opt)
    assert FSDP.get_state_dict_type(f).state_dict_type == StateDictType.FULL_STATE_DICT   # restored
    errs = []
    for sd, osd in ((full_sd, full_osd), (sh_sd, sh_osd)):
        g = FSDP(_net(4), **wrap)             # other initial weights
        gopt = torch.optim.AdamW(g.parameters(), lr=1e-2)
        g.load_state_dict(sd)
        gopt.load_state_dict(FSDP.optim_state_dict_to_load(g, gopt, osd))
        # one more identical step on both
        torch.manual_seed(70 + rank)
        x = torch.randn(4, 12)
        for model, o in ((g, gopt),):
            o.zero_grad()
            model(x).pow(2).mean().backward()
            o.step()
        ref = FSDP(_net(4), **wrap)
        ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
        ref.load_state_dict(full_sd)
        ropt.load_state_dict(FSDP.optim_state_dict_to_load(ref, ropt, full_osd))
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()
        a, b = g.state_dict(), ref.state_dict()
        errs.append(max(float((a[k] - b[k]).abs().max()) for k in a))
    # the sharded scaler: a non-finite gradient on ONE rank skips the step on every rank
    scaler = ShardedGradScaler(device="cpu", init_scale=4.0)
    before = {k: v.clone() for k, v in f.state_dict().items()}
    opt.zero_grad()
    loss = f(torch.randn(4, 12)).pow(2).mean()
    scaler.scale(loss).backward()
    if rank == 1:
        next(p for p in f.parameters() if p.grad is not None and p.grad.numel() > 0).grad.view(-1)[0] = float("inf")
    scaler.step(opt)
    scaler.update()
    after = f.state_dict()
    skipped = all(torch.equal(before[k], after[k]) for k in before)
    return errs, skipped, float(scaler.get_scale())


def test_fsdp1_state_dict_types_optim_state_and_sharded_scaler():
    for errs, skipped, scale in run_ranks(_state_dict_types_worker, 2):
        assert errs[0] < 1e-6 and errs[1] < 1e-6, errs   # loaded from the full form, from the sharded form
        assert skipped and scale == 2.0
