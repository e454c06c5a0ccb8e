"""GPipe and 1F1B over gloo ranks: gradients equal those of the un-pipelined model."""
import pytest
import torch
from torch import nn

from tests.distutil import run_ranks


def _make(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(4)])


def _worker(rank, world, sched_name, n_mb):
    from tensorplay_b200.distributed.pipelining import PipelineStage, Schedule1F1B, ScheduleGPipe
    full = _make()
    per = 4 // world
    sub = nn.Sequential(*[full[i] for i in range(rank * per, (rank + 1) * per)])
    stage = PipelineStage(sub, rank, world, device="cpu")
    loss_fn = lambda out, tgt: ((out - tgt) ** 2).mean()
    sched = {"gpipe": ScheduleGPipe, "1f1b": Schedule1F1B}[sched_name](stage, n_mb, loss_fn)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8, 16, generator=g)
    y = torch.randn(8, 16, generator=g)
    for it in range(2):  # second step reuses cached shapes
        for p in sub.parameters():
            p.grad = None
        losses = []
        if rank == 0:
            sched.step(x)
        elif rank == world - 1:
            sched.step(target=y, losses=losses)
        else:
            sched.step()
        ref = _make()
        loss_fn(ref(x), y).backward()
        for (n, p), q in zip(sub.named_parameters(), [q for i in range(rank * per, (rank + 1) * per) for q in ref[i].parameters()]):
            assert torch.allclose(p.grad, q.grad, atol=1e-6), (sched_name, rank, n)
        if rank == world - 1:
            assert len(losses) == n_mb
            assert abs(torch.stack(losses).mean().item() - loss_fn(ref(x), y).item()) < 1e-6
    return True


@pytest.mark.parametrize("sched,world,n_mb", [("gpipe", 2, 4), ("1f1b", 2, 4), ("1f1b", 4, 8), ("1f1b", 4, 2)])
def test_pipeline_schedules(sched, world, n_mb):
    assert all(run_ranks(_worker, world, sched, n_mb))


def _worker_interleaved(rank, world):
    from tensorplay_b200.distributed.pipelining import PipelineStage, ScheduleInterleaved1F1B
    full = _make()
    stages = [PipelineStage(full[s], s, 4, device="cpu") for s in range(4) if s % world == rank]
    loss_fn = lambda out, tgt: ((out - tgt) ** 2).mean()
    sched = ScheduleInterleaved1F1B(stages, 4, loss_fn)
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(8, 16, generator=g), torch.randn(8, 16, generator=g)
    if rank == 0:
        sched.step(x, target=None)
    else:
        sched.step(target=y)
    ref = _make()
    loss_fn(ref(x), y).backward()
    for st in stages:
        for p, q in zip(st.submod.parameters(), ref[st.stage_index].parameters()):
            assert torch.allclose(p.grad, q.grad, atol=1e-6)
    return True


def test_interleaved_two_ranks_four_stages():
    assert all(run_ranks(_worker_interleaved, 2))
