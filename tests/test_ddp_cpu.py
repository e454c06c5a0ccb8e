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
