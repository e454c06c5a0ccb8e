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


def _protocol_worker(rank, world, tmp):
    """De-duplicated replicated tensors, fully_shard state dicts by name (sharded and full), a resharding
    load through them, the Hugging Face layout and its consolidation."""
    import json
    import os
    import torch.distributed as dist
    from torch import nn
    import tensorplay_b200.distributed.checkpoint as dcp
    from tensorplay_b200.distributed.fsdp import fully_shard

    def make(seed):
        torch.manual_seed(seed)
        return nn.Sequential(nn.Linear(10, 7), nn.Tanh(), nn.Linear(7, 5))

    dense = make(0)
    m = make(0)
    fully_shard(m)
    opt = torch.optim.AdamW(m.parameters(), lr=0.1)
    m(torch.randn(3, 10)).sum().backward()
    opt.step()
    msd, osd = dcp.get_state_dict(m, opt)
    assert isinstance(msd["0.weight"], dcp.ShardedTensor) and msd["0.weight"].global_shape == (7, 10)
    assert set(osd["state"]) == {"0.weight", "0.bias", "2.weight", "2.bias"}
    big = torch.arange(1000.).reshape(10, 100)
    extra = {"a": big, "b": big + 1, "c": torch.ones(3), "step": 7}
    d1 = os.path.join(tmp, "sharded")
    dcp.save({"model": msd, "optim": osd, "extra": extra}, checkpoint_id=d1)
    with open(os.path.join(d1, ".metadata")) as f:
        meta = json.load(f)["state_dict_metadata"]
    owners = {meta[k]["rank"] for k in ("extra.a", "extra.b", "extra.c")}
    assert owners == set(range(world)), owners          # replicated tensors are spread over the ranks
    # load into a fresh model + optimizer through the same helpers
    m2 = make(1)
    fully_shard(m2)
    opt2 = torch.optim.AdamW(m2.parameters(), lr=0.1)
    m2(torch.randn(3, 10)).sum().backward()
    opt2.step()
    msd2, osd2 = dcp.get_state_dict(m2, opt2)
    got = {"model": msd2, "optim": osd2, "extra": {"a": torch.zeros(10, 100), "b": torch.zeros(10, 100),
                                                  "c": torch.zeros(3), "step": 0}}
    dcp.load(got, checkpoint_id=d1)
    dcp.set_state_dict(m2, opt2, model_state_dict=got["model"], optim_state_dict=got["optim"])
    assert got["extra"]["step"] == 7 and torch.equal(got["extra"]["b"], big + 1)
    full1 = dcp.get_model_state_dict(m, options=dcp.StateDictOptions(full_state_dict=True))
    full2 = dcp.get_model_state_dict(m2, options=dcp.StateDictOptions(full_state_dict=True))
    for k in full1:
        assert torch.equal(full1[k], full2[k]), k
        assert full1[k].shape == dict(dense.named_parameters())[k].shape
    fo1 = dcp.get_optimizer_state_dict(m, opt, options=dcp.StateDictOptions(full_state_dict=True))
    fo2 = dcp.get_optimizer_state_dict(m2, opt2, options=dcp.StateDictOptions(full_state_dict=True))
    assert torch.equal(fo1["state"]["2.weight"]["exp_avg"], fo2["state"]["2.weight"]["exp_avg"])
    assert fo1["state"]["2.weight"]["exp_avg"].shape == (5, 7)
    # a full state dict loads into a plain (unsharded) model and into the sharded one
    plain = make(5)
    dcp.set_model_state_dict(plain, full1)
    assert torch.equal(plain[0].weight, full1["0.weight"])
    m3 = make(6)
    fully_shard(m3)
    dcp.set_model_state_dict(m3, full1)
    assert torch.equal(dcp.get_model_state_dict(m3, options=dcp.StateDictOptions(full_state_dict=True))["2.weight"], full1["2.weight"])
    # Hugging Face layout from full tensors, and by consolidating the sharded checkpoint
    d2 = os.path.join(tmp, "hf")
    dcp.save(full1, storage_writer=dcp.HuggingFaceStorageWriter(d2))
    back = {k: torch.zeros_like(v) for k, v in full1.items()}
    dcp.load(back, storage_reader=dcp.HuggingFaceStorageReader(d2))
    assert all(torch.equal(back[k], full1[k]) for k in full1)
    with open(os.path.join(d2, "model.safetensors.index.json")) as f:
        assert len(set(json.load(f)["weight_map"].values())) == world
    dist.barrier()
    if rank == 0:
        d3 = os.path.join(tmp, "consolidated")
        dcp.consolidate_to_hf(d1, d3, max_shard_bytes=2000)
        merged = dcp.load_hf(d3)
        assert torch.equal(merged["model.0.weight"], full1["0.weight"]) and torch.equal(merged["extra.a"], big)
    dist.barrier()
    return True


def test_planner_state_dict_helpers_and_hf_layout(tmp_path):
    assert all(run_ranks(_protocol_worker, 2, str(tmp_path)))
