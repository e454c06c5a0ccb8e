"""Sharded engine on 2 gloo ranks (CPU): losses and parameters must match a dense run."""
import copy

import torch

from tests.distutil import run_ranks


def _worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine

    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128,
                           vocab_size=128, num_layers=3)
    base = Llama(cfg)
    base.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 16), generator=g)
    tgts = torch.randint(0, cfg.vocab_size, (world, 2, 16), generator=g)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    res = {}
    for ckpt in (True, False, "selective"):
        eng = FSDPEngine(copy.deepcopy(base), ocfg, comm="torch", activation_checkpointing=ckpt)
        losses = []
        for _ in range(4):
            l = eng.step(toks[rank], tgts[rank])
            dist.all_reduce(l)
            losses.append(float(l) / world)
        res[ckpt] = (losses, eng.gather_full_state())
    ref = copy.deepcopy(base)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_losses = []
    for _ in range(4):
        opt.zero_grad()
        loss = ref(toks.flatten(0, 1), tgts.flatten(0, 1))
        loss.backward()
        opt.step()
        ref_losses.append(float(loss.detach()))
    for ckpt in (True, False, "selective"):
        losses, state = res[ckpt]
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 1e-5, (ckpt, losses, ref_losses)
        for n, p in ref.named_parameters():
            d = (state[n] - p.detach()).abs().max().item()
            assert d < 2e-4, (n, d)
    return True


def test_engine_two_ranks_gloo_matches_dense():
    assert all(run_ranks(_worker, 2))


def _clip_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine

    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128,
                           vocab_size=128, num_layers=2)
    base = Llama(cfg)
    base.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 16), generator=g)
    tgts = torch.randint(0, cfg.vocab_size, (world, 2, 16), generator=g)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = FSDPEngine(copy.deepcopy(base), ocfg, comm="torch", max_grad_norm=0.05)
    norms = []
    for _ in range(3):
        eng.step(toks[rank], tgts[rank])
        norms.append(float(eng.grad_norm))
    state = eng.gather_full_state()
    ref = copy.deepcopy(base)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for i in range(3):
        opt.zero_grad()
        ref(toks.flatten(0, 1), tgts.flatten(0, 1)).backward()
        n = float(torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05))
        assert abs(n - norms[i]) < 1e-4 * max(1.0, n), (i, n, norms[i])
        opt.step()
    for n, p in ref.named_parameters():
        d = (state[n] - p.detach()).abs().max().item()
        assert d < 2e-4, (n, d)
    dist.barrier()
    return True


def test_engine_two_ranks_clipped_step():
    assert all(run_ranks(_clip_worker, 2))


def _ckpt_worker(rank, world, directory, phase):
    """phase 0: train 2 steps on `world` ranks and save; phase 1: load (possibly on another world
    size), train 2 more steps and return the final parameters."""
    import torch.distributed as dist
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine

    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128,
                           vocab_size=128, num_layers=2)
    base = Llama(cfg)
    base.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (4, 2, 2, 16), generator=g)  # [step, 2 micro-batches, B, T]
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = FSDPEngine(base, ocfg, comm="torch")
    per = 2 // world  # every world size sees the same global batch of 2 micro-batches per step

    def batch(step):
        x = toks[step, rank * per: (rank + 1) * per].flatten(0, 1)
        return x, x

    if phase == 0:
        for st in range(2):
            eng.step(*batch(st))
        eng.save_checkpoint(directory)
        return True
    eng.load_checkpoint(directory)
    assert eng.step_count == 2
    for st in range(2, 4):
        eng.step(*batch(st))
    state = eng.gather_full_state()
    return {k: v.numpy().copy() for k, v in state.items()}  # by value through the result queue


def test_engine_checkpoint_resume_and_reshard(tmp_path):
    d = str(tmp_path / "ckpt")
    assert all(run_ranks(_ckpt_worker, 2, d, 0))
    resumed2 = run_ranks(_ckpt_worker, 2, d, 1)[0]   # same world size
    resumed1 = run_ranks(_ckpt_worker, 1, d, 1)[0]   # resharded 2 -> 1
    # uninterrupted reference: 4 steps on one rank over the same global batches
    import copy as _copy
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128,
                           vocab_size=128, num_layers=2)
    ref = Llama(cfg)
    ref.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (4, 2, 2, 16), generator=g)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for st in range(4):
        opt.zero_grad()
        x = toks[st].flatten(0, 1)
        ref(x, x).backward()
        opt.step()
    for n, p in ref.named_parameters():
        for got in (resumed2, resumed1):
            d_ = (torch.from_numpy(got[n]) - p.detach()).abs().max().item()
            assert d_ < 3e-4, (n, d_)


def _hsdp_worker(rank, world):
    """2 x 2 hybrid sharding: shard over pairs {0,1}, {2,3}; replicate over {0,2}, {1,3}."""
    import torch.distributed as dist
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine

    shard_groups = [dist.new_group([0, 1]), dist.new_group([2, 3])]
    rep_groups = [dist.new_group([0, 2]), dist.new_group([1, 3])]
    shard_g, rep_g = shard_groups[rank // 2], rep_groups[rank % 2]
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128,
                           vocab_size=128, num_layers=2)
    base = Llama(cfg)
    base.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 16), generator=g)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    eng = FSDPEngine(copy.deepcopy(base), ocfg, group=shard_g, comm="torch", replicate_group=rep_g)
    for _ in range(3):
        eng.step(toks[rank], toks[rank])
    state = eng.gather_full_state()
    ref = copy.deepcopy(base)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(3):
        opt.zero_grad()
        ref(toks.flatten(0, 1), toks.flatten(0, 1)).backward()
        opt.step()
    for n, p in ref.named_parameters():
        d = (state[n] - p.detach()).abs().max().item()
        assert d < 2e-4, (n, d)
    dist.barrier()
    return True


def test_engine_hybrid_sharding_2x2():
    assert all(run_ranks(_hsdp_worker, 4))
