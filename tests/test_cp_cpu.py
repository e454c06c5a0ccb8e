"""Ring attention on two and three gloo ranks against full-sequence attention."""
import torch

from tests.distutil import run_ranks


def _worker(rank, world, causal):
    import torch.distributed as dist
    from tensorplay_b200.ops.attention import attention_reference
    from tensorplay_b200.parallel.cp import context_parallel_shard, context_parallel_unshard, ring_attention
    torch.manual_seed(0)
    B, T, Hq, Hkv, D = 2, 12 * world, 4, 2, 16
    q = torch.randn(B, T, Hq, D, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, requires_grad=True)
    v = torch.randn(B, T, Hkv, D, requires_grad=True)
    ref = attention_reference(q, k, v, causal)
    g = torch.randn_like(ref)
    ref.backward(g)
    ql, kl, vl, gl = (t.detach().requires_grad_() for t in context_parallel_shard([q, k, v, g], [1, 1, 1, 1]))
    out = ring_attention(ql, kl, vl, causal)
    out.backward(gl.detach())
    full, = context_parallel_unshard([out.detach()], [1])
    torch.testing.assert_close(full, ref.detach(), rtol=1e-4, atol=1e-5)
    for loc, glob in ((ql, q), (kl, k), (vl, v)):
        torch.testing.assert_close(loc.grad, glob.grad.chunk(world, dim=1)[rank], rtol=1e-4, atol=1e-5)
    dist.barrier()


def test_ring_attention_causal_two_ranks():
    run_ranks(_worker, 2, True)


def test_ring_attention_full_three_ranks():
    run_ranks(_worker, 3, False)


def _zigzag_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.ops.attention import attention_reference
    from tensorplay_b200.parallel.cp import _plan, context_parallel_shard, context_parallel_unshard, ring_attention
    torch.manual_seed(0)
    B, T, Hq, Hkv, D = 1, 8 * 2 * world, 4, 2, 16
    q = torch.randn(B, T, Hq, D, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, requires_grad=True)
    v = torch.randn(B, T, Hkv, D, requires_grad=True)
    ref = attention_reference(q, k, v, True)
    g = torch.randn_like(ref)
    ref.backward(g)
    ql, kl, vl, gl = (t.detach().requires_grad_() for t in
                      context_parallel_shard([q, k, v, g], [1, 1, 1, 1], load_balance=True))
    out = ring_attention(ql, kl, vl, True, load_balance=True)
    out.backward(gl.detach())
    full, = context_parallel_unshard([out.detach()], [1], load_balance=True)
    torch.testing.assert_close(full, ref.detach(), rtol=1e-4, atol=1e-5)
    for loc, glob in ((ql, q), (kl, k), (vl, v)):
        want, = context_parallel_shard([glob.grad], [1], load_balance=True)
        torch.testing.assert_close(loc.grad, want, rtol=1e-4, atol=1e-5)
    # balanced: every rank computes the same number of chunk pairs (2 * world + 1 with the two causal ones)
    pairs = sum(len(p) for _, p in _plan(rank, world, True, True))
    assert pairs == 2 * world + 1
    dist.barrier()


def test_ring_attention_load_balanced_causal():
    run_ranks(_zigzag_worker, 2)
    run_ranks(_zigzag_worker, 3)
