"""Qwen3-MoE-shaped model on CPU: routing and expert FFN against a per-token oracle, training through
the sharded engine, and expert parallelism over two gloo ranks against one rank."""
import copy

import torch

from tests.distutil import run_ranks


def _cfg(**kw):
    from tensorplay_b200.models.qwen3_moe import Qwen3MoEConfig
    base = dict(vocab_size=64, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                num_experts=4, moe_intermediate=16, top_k=2, max_seq_len=16)
    base.update(kw)
    return Qwen3MoEConfig.tiny(**base)


def test_routing_and_expert_ffn_match_per_token_oracle():
    from tensorplay_b200.parallel.moe import expert_parallel_ffn, topk_route
    g = torch.Generator().manual_seed(0)
    T, H, E, I, k = 12, 16, 4, 8, 2
    x = torch.randn(T, H, generator=g)
    logits = torch.randn(T, E, generator=g)
    wgu, wd = torch.randn(E, 2 * I, H, generator=g) * 0.2, torch.randn(E, H, I, generator=g) * 0.2
    idx, w, aux = topk_route(logits, k)
    torch.testing.assert_close(w.sum(-1), torch.ones(T))
    probs = torch.softmax(logits, -1)
    assert torch.equal(idx, probs.topk(k, -1).indices)
    # balanced routing gives aux = 1; routing everything to one expert gives the maximum E
    uniform = topk_route(torch.zeros(4 * E, E) + torch.eye(E).repeat(4, 1) * 1e-3, 1)[2]
    assert abs(uniform.item() - 1.0) < 1e-2
    collapsed = topk_route(torch.tensor([[10.0, 0, 0, 0]]).repeat(8, 1), 1)[2]
    assert collapsed.item() > 3.9
    y = expert_parallel_ffn(x, idx, w, wgu, wd)
    ref = torch.zeros(T, H)
    for t in range(T):
        for s in range(k):
            e = int(idx[t, s])
            h = wgu[e] @ x[t]
            ref[t] += w[t, s] * (wd[e] @ (torch.nn.functional.silu(h[:I]) * h[I:]))
    torch.testing.assert_close(y, ref, rtol=1e-4, atol=1e-5)


def test_model_trains_through_the_engine():
    from tensorplay_b200.models.qwen3_moe import Qwen3MoE
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine
    cfg = _cfg()
    m = Qwen3MoE(cfg)
    m.reset_parameters(seed=0)
    eng = FSDPEngine(m, AdamWConfig(lr=3e-3))
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab_size, (2, 12), generator=g)
    losses = [float(eng.step(tok[:, :-1], tok[:, 1:])) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.2                    # the fixed batch is being fitted


def _ep_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.models.qwen3_moe import Qwen3MoE
    cfg = _cfg(aux_loss_coef=0.0)
    solos = [dist.new_group([r]) for r in range(world)]    # every rank creates every group
    full = Qwen3MoE(cfg, ep_group=solos[rank])             # all experts on one rank: the oracle
    full.reset_parameters(seed=0)
    ep = Qwen3MoE(cfg, ep_group=dist.group.WORLD)          # experts split over the two ranks
    El = cfg.num_experts // world
    with torch.no_grad():
        for le, lf in zip(ep.layers, full.layers):
            for n, p in le.named_parameters():
                src = dict(lf.named_parameters())[n]
                p.copy_(src[rank * El: (rank + 1) * El] if n in ("w_gate_up", "w_down") else src)
        ep.embed.copy_(full.embed)
        ep.final_norm.copy_(full.final_norm)
        ep.lm_head.copy_(full.lm_head)
    assert ep.layers[0].w_gate_up.shape[0] == El
    g = torch.Generator().manual_seed(2 + rank)            # every rank its own tokens
    tok = torch.randint(0, cfg.vocab_size, (2, 10), generator=g)
    l_ep = ep(tok[:, :-1], tok[:, 1:])
    l_full = full(tok[:, :-1], tok[:, 1:])
    torch.testing.assert_close(l_ep, l_full, rtol=1e-5, atol=1e-6)
    l_ep.backward()
    l_full.backward()
    # a local expert's gradient collects the tokens of both ranks: sum the oracle's over ranks
    want = full.layers[1].w_down.grad.clone()
    dist.all_reduce(want)
    torch.testing.assert_close(ep.layers[1].w_down.grad, want[rank * El: (rank + 1) * El], rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(ep.layers[0].router.grad, full.layers[0].router.grad, rtol=1e-4, atol=1e-6)
    dist.barrier()
    return True


def test_expert_parallel_two_ranks_equals_single_rank_experts():
    assert all(run_ranks(_ep_worker, 2))
