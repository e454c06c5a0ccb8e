"""Distributed components that had no direct test, on gloo ranks: device mesh, ZeRO-1 optimizer,
DDP communication hooks (bf16 compression, PowerSGD), Join, loss-parallel cross-entropy, sequence
parallel gradient sync."""
import copy

import torch
from torch import nn as tnn

from tests.distutil import run_ranks


def _mesh_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.device_mesh import init_device_mesh
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    tp_g, dp_g = mesh.get_group("tp"), mesh.get_group("dp")
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=tp_g)                     # tp pairs: {0,1}, {2,3}
    assert t.item() == (1.0 if rank < 2 else 5.0)
    t = torch.tensor([float(rank)])
    dist.all_reduce(t, group=dp_g)                     # dp pairs: {0,2}, {1,3}
    assert t.item() == (2.0 if rank % 2 == 0 else 4.0)
    assert mesh["tp"].size() == 2 and mesh.get_local_rank("tp") == rank % 2
    return True


def test_device_mesh_2d_groups():
    assert all(run_ranks(_mesh_worker, 4))


def _zero_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer
    torch.manual_seed(0)
    model = tnn.Sequential(tnn.Linear(8, 16), tnn.Tanh(), tnn.Linear(16, 4))
    ref = copy.deepcopy(model)
    zo = ZeroRedundancyOptimizer(model.parameters(), optimizer_class=torch.optim.AdamW, lr=1e-2)
    ro = torch.optim.AdamW(ref.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(1)
    for _ in range(3):
        x = torch.randn(world, 4, 8, generator=g)
        for m, o, data in ((model, zo, x[rank]), (ref, ro, x.flatten(0, 1))):
            o.zero_grad()
            m(data).pow(2).mean().backward()
            if m is model:
                for p in m.parameters():
                    dist.all_reduce(p.grad)
                    p.grad.div_(world)
            o.step()
    for a, b in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # each rank holds optimizer state for its partition only
    assert 0 < len(zo.optim.state) < len(list(model.parameters()))
    return True


def test_zero_redundancy_optimizer_matches_full_optimizer():
    assert all(run_ranks(_zero_worker, 2))


def _hooks_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed import algorithms as A
    from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP
    torch.manual_seed(0)
    base = tnn.Sequential(tnn.Linear(32, 32, bias=False), tnn.Tanh(), tnn.Linear(32, 8, bias=False))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(world, 16, 32, generator=g)
    ref = copy.deepcopy(base)
    ref(x.flatten(0, 1)).pow(2).mean().backward()
    want = [p.grad.clone() for p in ref.parameters()]
    # bf16 compression: the averaged gradient within bf16 rounding
    m = DDP(copy.deepcopy(base))
    m.register_comm_hook(None, A.bf16_compress_hook)
    m(x[rank]).pow(2).mean().backward()
    for p, w in zip(m.parameters(), want):
        torch.testing.assert_close(p.grad, w, rtol=2e-2, atol=2e-3)
    # PowerSGD at full rank reproduces the average; at rank 2 the error feedback holds the rest
    for r, exact in ((32, True), (2, False)):
        m = DDP(copy.deepcopy(base), bucket_cap_mb=1e-3)      # one parameter per bucket
        state = {"process_group": None, "rank": r}
        m.register_comm_hook(state, A.powerSGD_hook)
        m(x[rank]).pow(2).mean().backward()
        p0, w0 = next(iter(m.parameters())), want[0]
        same = torch.tensor([float(p0.grad.sum())])
        both = [torch.zeros(1) for _ in range(world)]
        dist.all_gather(both, same)
        assert abs(both[0].item() - both[1].item()) < 1e-5         # identical result on every rank
        if exact:
            torch.testing.assert_close(p0.grad, w0, rtol=1e-3, atol=1e-5)
        else:
            assert (p0.grad - w0).norm() < w0.norm() and len(state["err"]) > 0
    return True


def test_ddp_comm_hooks():
    assert all(run_ranks(_hooks_worker, 2))


def _join_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.algorithms import Join
    from torch.nn.parallel import DistributedDataParallel as TorchDDP
    torch.manual_seed(0)
    m = TorchDDP(tnn.Linear(4, 2))
    n_batches = 3 + rank                                     # uneven inputs
    with Join([m]):
        for _ in range(n_batches):
            m(torch.randn(2, 4)).sum().backward()
    dist.barrier()
    return n_batches


def test_join_with_uneven_inputs():
    assert run_ranks(_join_worker, 2) == [3, 4]


def _loss_parallel_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.tensor.parallel import (SequenceParallel, loss_parallel, parallelize_module,
                                                             sync_replicated_grads)
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(10, 16, generator=g)
    target = torch.randint(0, 16, (10,), generator=g)
    full = logits.clone().requires_grad_()
    ref = torch.nn.functional.cross_entropy(full, target)
    ref.backward()
    shard = logits[:, rank * 8: (rank + 1) * 8].clone().requires_grad_()
    with loss_parallel() as lp:
        loss = lp.cross_entropy(shard, target)
    loss.backward()
    torch.testing.assert_close(loss, ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(shard.grad, full.grad[:, rank * 8: (rank + 1) * 8], rtol=1e-5, atol=1e-6)
    # sequence parallel: a norm sees its rows only; the synchronised gradient is the full one
    norm = tnn.LayerNorm(6)
    wrap = tnn.Sequential(norm)
    parallelize_module(wrap, None, {"0": SequenceParallel()})
    x = torch.randn(8, 6, generator=g)
    dense = tnn.LayerNorm(6)
    dense(x).pow(3).sum().backward()
    wrap(x[rank * 4: (rank + 1) * 4]).pow(3).sum().backward()
    sync_replicated_grads(wrap)
    torch.testing.assert_close(norm.weight.grad, dense.weight.grad, rtol=1e-4, atol=1e-5)
    dist.barrier()
    return True


def test_loss_parallel_and_sequence_parallel():
    assert all(run_ranks(_loss_parallel_worker, 2))


def _funcol_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed import _functional_collectives as fc
    from tensorplay_b200.distributed import _symmetric_memory as sm
    x = torch.arange(4.0) + 10 * rank
    g = fc.all_gather_single(x, 0, dist.group.WORLD)
    assert fc.wait_tensor(g).tolist() == [0, 1, 2, 3, 10, 11, 12, 13]
    r = fc.wait_tensor(fc.reduce_scatter_single(torch.ones(4) * (rank + 1), "sum", 0, dist.group.WORLD))
    assert r.tolist() == [3.0, 3.0]
    xa = (torch.ones(2) * (rank + 1)).requires_grad_()
    ga = fc.all_gather_single_autograd(xa, 0, dist.group.WORLD)
    fc.wait_tensor(ga).pow(2).sum().backward()
    assert xa.grad.tolist() == [4.0 * (rank + 1)] * 2      # every rank's loss sees this shard: 2 x (2 x)
    out = torch.zeros(2)
    fc.reduce_scatter_inplace(out, torch.arange(4.0))
    assert out.tolist() == ([0.0, 2.0] if rank == 0 else [4.0, 6.0])
    buf = torch.zeros(3)
    works = fc.batch_p2p_ops_inplace([("send", torch.full((3,), float(rank)), 1 - rank), ("recv", buf, 1 - rank)])
    for w in works:
        w.wait()
    assert buf.tolist() == [float(1 - rank)] * 3
    # uneven reduce-scatter and n-d all-to-all of the symmetric-memory surface (plain collectives on CPU)
    inp = torch.arange(10.0).view(5, 2) * (rank + 1)
    mine = sm.reduce_scatter_offset(inp, offsets=[2, 5])
    want = (torch.arange(10.0).view(5, 2) * 3)[:2] if rank == 0 else (torch.arange(10.0).view(5, 2) * 3)[2:]
    torch.testing.assert_close(mine, want)
    a2a = sm.all_to_all_nd(torch.full((2, 2, 2), float(rank)))
    assert a2a[0].unique().tolist() == [0.0] and a2a[1].unique().tolist() == [1.0]
    assert sm.get_backend() in ("vmm", "ipc") and sm.get_signal_pad_size() > 0
    dist.barrier()
    return True


def test_functional_collective_spellings_and_symmetric_memory_helpers():
    assert all(run_ranks(_funcol_worker, 2))


def _extras_worker(rank, world):
    import torch.distributed as dist
    import tensorplay_b200.distributed as tpd

    # gather into one tensor on a destination rank
    t = torch.full((3,), float(rank))
    out = torch.empty(world, 3) if rank == 1 else None
    tpd.gather_single(t, out, dst=1)
    if rank == 1:
        assert out.tolist() == [[float(r)] * 3 for r in range(world)]
    # coalesced all-gather: two dtypes, three tensors, one collective per dtype
    ins = [torch.arange(4.0) + rank, torch.tensor([rank], dtype=torch.int64), torch.full((2, 2), float(rank))]
    outs = [torch.empty(world * 4), torch.empty(world, dtype=torch.int64), torch.empty(world, 2, 2)]
    tpd.all_gather_single_coalesced(outs, ins)
    assert outs[0].view(world, 4)[1].tolist() == [1.0, 2.0, 3.0, 4.0] and outs[1].tolist() == list(range(world))
    assert outs[2][1].tolist() == [[1.0, 1.0], [1.0, 1.0]]
    work = tpd.all_gather_single_coalesced(outs, ins, async_op=True)
    work.wait()
    assert outs[1].tolist() == list(range(world))
    # coalesced reduce-scatter, both spellings
    ins = [torch.arange(2.0 * world) * (rank + 1), torch.ones(world * 3) * (rank + 1)]
    outs = [torch.empty(2), torch.empty(3)]
    tpd.reduce_scatter_single_coalesced(outs, ins)
    tot = sum(range(1, world + 1))
    assert outs[0].tolist() == [2.0 * rank * tot, (2.0 * rank + 1) * tot] and outs[1].tolist() == [float(tot)] * 3
    outs2 = [torch.empty(2)]
    tpd.reduce_scatter_coalesced(outs2, [[torch.full((2,), float(rank + r)) for r in range(world)]])
    assert outs2[0].tolist() == [float(sum(q + rank for q in range(world)))] * 2
    # names of communication regions and the timeout setter
    with tpd.record_comm("grad-bucket-3"):
        from tensorplay_b200.distributed._collective_extras import current_comm_name
        assert current_comm_name() == "grad-bucket-3"
        dist.barrier()
    assert current_comm_name() is None
    from datetime import timedelta
    tpd.set_timeout(timedelta(seconds=120))
    assert tpd.SHRINK_DEFAULT == 0 and tpd.SHRINK_ABORT == 1 and tpd.AllgatherOptions is not None
    return True


def test_collective_spellings_beyond_pytorchs():
    assert all(run_ranks(_extras_worker, 2))
