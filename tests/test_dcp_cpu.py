"""Distributed checkpoint: save on 2 ranks, load on 1 and on 3 (resharding); engine resume."""
import copy
import os

import torch

from tests.distutil import run_ranks


def _global():
    g = torch.Generator().manual_seed(0)
    return torch.randn(10, 6, generator=g), torch.arange(5.0)


def _shard(t, world, rank):
    c = (t.shape[0] + world - 1) // world
    lo, hi = min(rank * c, t.shape[0]), min((rank + 1) * c, t.shape[0])
    return t[lo:hi].clone(), lo


def _save(rank, world, path):
    from tensorplay_b200.distributed import checkpoint as dcp
    w, b = _global()
    local, lo = _shard(w, world, rank)
    sd = {"model": {"w": dcp.ShardedTensor(local, tuple(w.shape), (lo, 0)), "b": b.clone()}, "step": 7}
    fut = dcp.async_save(sd, checkpoint_id=path)
    fut.result(timeout=60)
    import torch.distributed as dist
    dist.barrier()
    return True


def _load(rank, world, path):
    from tensorplay_b200.distributed import checkpoint as dcp
    w, b = _global()
    local, lo = _shard(w, world, rank)
    sd = {"model": {"w": dcp.ShardedTensor(torch.zeros_like(local), tuple(w.shape), (lo, 0)), "b": torch.zeros(5)},
          "step": 0}
    dcp.load(sd, checkpoint_id=path)
    assert torch.equal(sd["model"]["w"].local, local) and torch.equal(sd["model"]["b"], b) and sd["step"] == 7
    return True


def test_dcp_reshard(tmp_path):
    path = str(tmp_path / "ckpt")
    assert all(run_ranks(_save, 2, path))
    assert os.path.exists(os.path.join(path, ".metadata")) and os.path.exists(os.path.join(path, "__1_0.distcp"))
    assert all(run_ranks(_load, 3, path))
    # single process, whole tensor
    from tensorplay_b200.distributed import checkpoint as dcp
    w, _ = _global()
    sd = {"model": {"w": torch.zeros(10, 6), "b": torch.zeros(5)}, "step": 0}
    dcp.load(sd, checkpoint_id=path)
    assert torch.equal(sd["model"]["w"], w)


def test_engine_checkpoint_resume(tmp_path):
    from tensorplay_b200.distributed import checkpoint as dcp
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=128, vocab_size=128)
    base = Llama(cfg)
    base.reset_parameters(0)
    tok = torch.randint(0, 128, (2, 16))
    e1 = FSDPEngine(copy.deepcopy(base), AdamWConfig(lr=1e-3))
    for _ in range(3):
        e1.step(tok, tok)
    dcp.save(dcp.engine_state_dict(e1), checkpoint_id=str(tmp_path / "eng"))
    cont = [float(e1.step(tok, tok)) for _ in range(2)]
    e2 = FSDPEngine(copy.deepcopy(base), AdamWConfig(lr=1e-3))
    dcp.load_engine_state_dict(e2, str(tmp_path / "eng"))
    resumed = [float(e2.step(tok, tok)) for _ in range(2)]
    assert resumed == cont
