"""The CPU toy-LLM configuration: decoder-only transformer (2 layers, d_model 128, 4 heads, LayerNorm,
GELU MLP 4x, learned positions, tied embeddings, vocab 512), context 64, batch 8, AdamW lr 3e-4
betas (0.9, 0.95) wd 0.1, 20 steps, fp32, seed 0. Single process vs ``fully_shard`` on 2 gloo
ranks: losses must agree to 1e-5."""
import torch

from tests.distutil import run_ranks

STEPS = 20


def _data(cfg):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, cfg.vocab_size, (STEPS, 8, cfg.n_ctx + 1), generator=g)


def _single():
    from tensorplay_b200.models.gpt2 import GPT2, GPT2Config
    cfg = GPT2Config.toy()
    torch.manual_seed(0)
    m = GPT2(cfg)
    m.reset_parameters(0)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    data = _data(cfg)
    losses = []
    for s in range(STEPS):
        opt.zero_grad()
        loss = m(data[s, :, :-1], data[s, :, 1:])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def _fsdp_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.distributed.fsdp import fully_shard
    from tensorplay_b200.models.gpt2 import GPT2, GPT2Config
    cfg = GPT2Config.toy()
    torch.manual_seed(0)
    m = GPT2(cfg)
    m.reset_parameters(0)
    for layer in m.layers:
        fully_shard(layer)
    fully_shard(m)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    data = _data(cfg)
    per = 8 // world
    losses = []
    for s in range(STEPS):
        opt.zero_grad()
        x = data[s, rank * per: (rank + 1) * per]
        loss = m(x[:, :-1], x[:, 1:])
        loss.backward()
        opt.step()
        l = loss.detach().clone()
        dist.all_reduce(l)
        losses.append(l.item() / world)
    return losses


def test_toy_llm_fsdp_two_ranks_matches_single_process():
    ref = _single()
    assert ref[-1] < ref[0]
    out = run_ranks(_fsdp_worker, 2)
    for losses in out:
        for a, b in zip(losses, ref):
            assert abs(a - b) < 1e-5, (losses, ref)
