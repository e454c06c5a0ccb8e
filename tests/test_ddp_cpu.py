"""DDP bucketed reducer on gloo ranks: gradients equal the dense average; no_sync accumulates."""
import torch

from tests.distutil import run_ranks


def _worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP
    from tensorplay_b200.models.gpt2 import GPT2, GPT2Config

    torch.manual_seed(rank)  # different init per rank: the ctor must broadcast rank 0's
    cfg = GPT2Config.toy()
    model = GPT2(cfg)
    model.reset_parameters(rank)
    ddp = DDP(model, bucket_cap_mb=0.05)
    assert len(ddp.buckets) > 2
    g = torch.Generator().manual_seed(3)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 8, 16), generator=g)
    # dense reference: same weights, whole batch
    ref = GPT2(cfg)
    ref.load_state_dict(model.state_dict())
    loss = ddp(toks[rank, 0], toks[rank, 0])
    loss.backward()
    ddp.synchronize()
    rl = ref(toks[:, 0].flatten(0, 1), toks[:, 0].flatten(0, 1))
    rl.backward()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-6), n
    # no_sync: local accumulation only, then a synced step reduces the sum
    for p in model.parameters():
        p.grad.zero_()
    for p in ref.parameters():
        p.grad = None
    with ddp.no_sync():
        ddp(toks[rank, 0], toks[rank, 0]).backward()
    ddp(toks[rank, 1], toks[rank, 1]).backward()
    ddp.synchronize()
    (ref(toks[:, 0].flatten(0, 1), toks[:, 0].flatten(0, 1)) + ref(toks[:, 1].flatten(0, 1), toks[:, 1].flatten(0, 1))).backward()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad, q.grad, atol=2e-6), n
    # comm hook contract
    calls = []

    def hook(state, bucket):
        calls.append(bucket.index())
        t = bucket.buffer().clone()
        dist.all_reduce(t)
        fut = torch.futures.Future()
        fut.set_result(t / world)
        return fut
    ddp.register_comm_hook(None, hook)
    for p in model.parameters():
        p.grad.zero_()
    ddp(toks[rank, 0], toks[rank, 0]).backward()
    assert sorted(calls) == list(range(len(ddp.buckets)))
    return True


def test_ddp_two_ranks():
    assert all(run_ranks(_worker, 2))


def _unused_worker(rank, world):
    import pytest
    from torch import nn
    from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.used = nn.Linear(6, 6)
            self.skipped = nn.Linear(6, 6)   # takes part in the forward only on rank 0
            self.head = nn.Linear(6, 2)

        def forward(self, x, use_skipped):
            h = torch.tanh(self.used(x))
            if use_skipped:
                h = h + self.skipped(x)
            return self.head(h)

    torch.manual_seed(0)
    x = torch.randn(world, 4, 6)
    m = Net()
    ddp = DDP(m, bucket_cap_mb=1e-4, find_unused_parameters=True)   # tiny buckets: one per parameter
    ddp(x[rank], rank == 0).sum().backward()
    ddp.synchronize()
    ref = Net()
    ref.load_state_dict(m.state_dict())
    sum(ref(x[r], r == 0).sum() for r in range(world)).backward()
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.grad, q.grad / world, atol=1e-6), n
    # without the flag an unfinished bucket is reported instead of being skipped silently
    strict = DDP(Net(), bucket_cap_mb=1e-4)
    with pytest.raises(RuntimeError, match="find_unused_parameters"):
        strict(x[rank], False).sum().backward()
    with pytest.raises(NotImplementedError):
        DDP(Net(), dim=1)
    return True


def test_ddp_unused_parameters_are_reduced_as_zeros_or_reported():
    assert all(run_ranks(_unused_worker, 2))
