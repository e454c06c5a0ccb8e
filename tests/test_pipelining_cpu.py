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
    from tensorplay_b200.distributed.pipelining import PipelineStage, ScheduleLoopedBFS
    full = _make()
    stages = [PipelineStage(full[s], s, 4, device="cpu") for s in range(4) if s % world == rank]
    loss_fn = lambda out, tgt: ((out - tgt) ** 2).mean()
    sched = ScheduleLoopedBFS(stages, 4, loss_fn)
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


def _make_deep(n_stages, seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(*[nn.Sequential(nn.Linear(16, 16), nn.Tanh()) for _ in range(n_stages)])


def _worker_runtime(rank, world, name, n_stages, n_mb, tmp):
    import tensorplay_b200.distributed.pipelining as pp
    full = _make_deep(n_stages)
    place = pp.v_placement(world) if name in ("zbv", "dualpipev") else pp.loop_placement(world)
    stages = [pp.PipelineStage(full[s], s, n_stages, device="cpu") for s in range(n_stages) if place(s) == rank]
    loss_fn = lambda out, tgt: ((out - tgt) ** 2).mean()
    if name == "csv":
        # a hand-written table: all forwards depth-first, then split backwards with the weight passes last
        if rank == 0:
            order = pp.interleaved_1f1b_order(world, n_stages // world, n_mb, split_backward=True)
            ref_sched = pp.PipelineScheduleRuntime(stages, n_mb, loss_fn, order=order, fill_with_weight=True, max_pending_w=2)
            ref_sched.dump_csv(tmp)
        import torch.distributed as dist
        dist.barrier()
        sched = pp.ScheduleFromCSV(stages, n_mb, loss_fn, csv_path=tmp)
        kinds = {a.kind for acts in sched.order.values() for a in acts}
        assert kinds == {"F", "I", "W"}
    else:
        cls = {"interleaved": pp.ScheduleInterleaved1F1B, "zb": pp.ScheduleInterleavedZeroBubble,
               "zbv": pp.ScheduleZBVZeroBubble, "dualpipev": pp.ScheduleDualPipeV}[name]
        sched = cls(stages, n_mb, loss_fn)
    g = torch.Generator().manual_seed(1)
    x, y = torch.randn(2 * n_mb, 16, generator=g), torch.randn(2 * n_mb, 16, generator=g)
    has_first, has_last = place(0) == rank, place(n_stages - 1) == rank
    for it in range(2):
        for st in stages:
            for p in st.submod.parameters():
                p.grad = None
        losses = []
        args = (x,) if has_first else ()
        sched.step(*args, target=y if has_last else None, losses=losses if has_last else None)
        ref = _make_deep(n_stages)
        loss_fn(ref(x), y).backward()
        for st in stages:
            for p, q in zip(st.submod.parameters(), ref[st.stage_index].parameters()):
                assert torch.allclose(p.grad, q.grad, atol=1e-6), (name, rank, st.stage_index)
        if has_last:
            assert abs(torch.stack(losses).mean().item() - loss_fn(ref(x), y).item()) < 1e-6
    # the depth-first order bounds the activations alive on a rank; breadth-first keeps the whole batch
    alive = worst = 0
    for a in sched.order[rank]:
        alive += 1 if a.kind == "F" else (-1 if a.kind in ("B", "I") else 0)
        worst = max(worst, alive)
    return worst, sched.bubble_fraction()


@pytest.mark.parametrize("name,world,n_stages,n_mb", [("interleaved", 2, 4, 4), ("interleaved", 4, 8, 8), ("zb", 2, 4, 4),
                                                      ("zb", 4, 8, 4), ("zbv", 2, 4, 4), ("zbv", 4, 8, 8),
                                                      ("dualpipev", 2, 4, 6), ("csv", 2, 4, 4)])
def test_runtime_schedules_match_the_dense_model(name, world, n_stages, n_mb, tmp_path):
    out = run_ranks(_worker_runtime, world, name, n_stages, n_mb, str(tmp_path / "sched.csv"))
    local = n_stages // world
    for rank, (worst, bubble) in enumerate(out):
        if name == "interleaved":
            assert worst <= 2 * (world - rank - 1) + (local - 1) * world + 1 < local * n_mb + 1 or n_mb <= world
        assert bubble < 0.5


def test_schedule_tables_are_consistent_without_ranks():
    """Every action appears once, dependencies hold tick by tick, transfers connect the right ranks."""
    import tensorplay_b200.distributed.pipelining as pp
    for order, S, place, fill in (
            (pp.interleaved_1f1b_order(4, 2, 8), 8, pp.loop_placement(4), False),
            (pp.interleaved_1f1b_order(4, 3, 8, split_backward=True), 12, pp.loop_placement(4), True),
            (pp.greedy_zero_bubble_order(8, pp.v_placement(4), 8, 8, 8), 8, pp.v_placement(4), False)):
        ticks = pp.simulate(order, S, place, fill, 8)
        seen = {}
        for t, tick in enumerate(ticks):
            for r, a in tick.actions.items():
                assert place(a.stage) == r and (a.stage, a.kind, a.mb) not in seen
                seen[(a.stage, a.kind, a.mb)] = t
            for src, dst, kind, stage, mb in tick.transfers:
                assert place(stage) == dst and src != dst
        for (s, k, m), t in seen.items():
            if k == "F" and s > 0:
                assert seen[(s - 1, "F", m)] < t
            if k in ("B", "I"):
                assert seen[(s, "F", m)] < t
                if s < S - 1:
                    assert seen.get((s + 1, "B", m), seen.get((s + 1, "I", m))) < t
            if k == "W":
                assert seen[(s, "I", m)] < t
        n_f = sum(1 for key in seen if key[1] == "F")
        assert n_f == S * 8
    with pytest.raises(ValueError):
        pp.interleaved_1f1b_order(4, 2, 6)


# ------------------------------------------------------------------ graph-splitting front end
class _Block(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.fc = nn.Linear(d, d)

    def forward(self, x):
        # a branch on a tensor property: blocks stay opaque calls, so this never meets the tracer
        if x.dtype == torch.float64:
            x = x.float()
        return x + torch.tanh(self.fc(x))


class _TinyLM(nn.Module):
    def __init__(self, d=16, n=4, vocab=32):
        super().__init__()
        self.embed = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList([_Block(d) for _ in range(n)])
        self.norm = nn.LayerNorm(d)
        self.head = nn.Linear(d, vocab)

    def forward(self, ids):
        x = self.embed(ids)
        for l in self.layers:
            x = l(x)
        return self.head(self.norm(x))


def test_pipeline_frontend_splits_and_composes():
    import tensorplay_b200.distributed.pipelining as pp
    torch.manual_seed(0)
    m = _TinyLM()
    ids = torch.randint(0, 32, (2, 8))
    pipe = pp.pipeline(m, (ids,), split_spec={"layers.1": pp.SplitPoint.END, "layers.3": pp.SplitPoint.BEGINNING})
    assert pipe.num_stages == 3
    assert torch.allclose(pipe(ids), m(ids), atol=1e-6)
    x = ids
    for i in range(3):
        x = pipe.get_stage_module(i)(x)
    assert torch.allclose(x, m(ids), atol=1e-6)
    # parameters are shared with the original model and every one lands in exactly one stage
    names = [n for i in range(3) for n, _ in pipe.get_stage_module(i).named_parameters()]
    assert len(names) == len(list(m.parameters()))
    st = pipe.build_stage(1)
    assert st.in_meta == ((2, 8, 16), torch.float32) and st.out_meta == ((2, 8, 16), torch.float32)
    with pytest.raises(ValueError):
        pp.pipeline(m, (ids,), split_spec={"layers.9": pp.SplitPoint.BEGINNING})


def test_pipeline_frontend_marker_and_refused_cut():
    import tensorplay_b200.distributed.pipelining as pp
    from tensorplay_b200.distributed.pipelining import pipe_split

    class Marked(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(8, 8), nn.Linear(8, 8)

        def forward(self, x):
            x = torch.relu(self.a(x))
            pipe_split()
            return self.b(x)

    torch.manual_seed(1)
    m = Marked()
    x = torch.randn(4, 8)
    pipe = pp.pipeline(m, (x,))
    assert pipe.num_stages == 2 and torch.allclose(pipe(x), m(x))

    class Skip(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(8, 8), nn.Linear(8, 8)

        def forward(self, x):
            h = self.a(x)
            return self.b(h) + x          # x crosses the cut beside h

    with pytest.raises(NotImplementedError):
        pp.pipeline(Skip(), (x,), split_spec={"b": pp.SplitPoint.BEGINNING})


def _worker_frontend(rank, world):
    import tensorplay_b200.distributed.pipelining as pp
    torch.manual_seed(0)
    m = _TinyLM()
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 32, (8, 8), generator=g)
    tgt = torch.randint(0, 32, (8, 8), generator=g)
    pipe = pp.pipeline(m, (ids[:2],), split_spec={"layers.2": pp.SplitPoint.BEGINNING})
    stage = pipe.build_stage(rank, device="cpu")
    loss_fn = lambda out, t: torch.nn.functional.cross_entropy(out.reshape(-1, 32), t.reshape(-1))
    sched = pp.Schedule1F1B(stage, 4, loss_fn)
    losses = []
    if rank == 0:
        sched.step(ids)
    else:
        sched.step(target=tgt, losses=losses)
    torch.manual_seed(0)
    ref = _TinyLM()
    loss_fn(ref(ids), tgt).backward()
    refp = dict(ref.named_parameters())
    checked = 0
    for n, p in m.named_parameters():
        if p.grad is not None:
            assert torch.allclose(p.grad, refp[n].grad, atol=1e-5), n
            checked += 1
    assert checked > 0
    return True


def test_pipeline_frontend_runs_under_1f1b():
    assert all(run_ranks(_worker_frontend, 2))
