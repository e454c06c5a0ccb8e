"""Single-process components that had no direct test: Muon, cache kinds, quantised linears, metric
collection, format conversion, FLOP counter, TensorBoard writer, prefetcher, memory plan."""
import os

import torch
from torch import nn as tnn

import tensorplay_b200 as tp
from tensorplay_b200 import metrics, nn, optim, quantization as Q


def test_muon_orthogonalises_and_trains():
    from tensorplay_b200.optim.muon import newton_schulz
    g = torch.randn(32, 48, generator=torch.Generator().manual_seed(0))
    o = newton_schulz(g, steps=8).float()
    sv = torch.linalg.svdvals(o)
    assert sv.max() < 1.3 and sv.min() > 0.3          # singular values pulled towards 1
    torch.manual_seed(0)
    lin = tnn.Linear(16, 16, bias=False)
    opt = optim.Muon([lin.weight], lr=0.05)
    x, y = torch.randn(64, 16), torch.randn(64, 16)
    first = None
    for _ in range(30):
        loss = (lin(x) - y).pow(2).mean()
        first = first or loss.item()
        opt.zero_grad()
        loss.backward()
        opt.step()
    assert loss.item() < 0.8 * first
    import pytest
    with pytest.raises(ValueError):
        b = tnn.Parameter(torch.zeros(4))
        b.grad = torch.ones(4)
        optim.Muon([b]).step()


def test_sliding_and_quantised_caches():
    k = torch.randn(1, 2, 10, 8)
    sw = nn.SlidingWindowCache(4)
    sw.update(k[:, :, :6], k[:, :, :6])
    kk, _ = sw.update(k[:, :, 6:7], k[:, :, 6:7])
    assert sw.get_seq_length() == 7 and sw.get_window_length() == 4 and kk.shape[2] == 5
    torch.testing.assert_close(kk[:, :, -1], k[:, :, 6])
    qc = nn.QuantizedCache()
    a, _ = qc.update(k[:, :, :5], k[:, :, :5])
    b, _ = qc.update(k[:, :, 5:], k[:, :, 5:])
    assert qc.get_seq_length() == 10 and b.shape == k.shape
    assert (b - k).abs().max() < k.abs().max() / 100     # int8 per (token, head): < 1 % of the range
    # a decoder produces (nearly) the same greedy tokens through the int8 cache
    torch.manual_seed(0)
    m = nn.DecoderLM(40, 32, 2, 4, 2)
    t = torch.randint(0, 40, (1, 6))
    ref = nn.generate(m, t, max_new_tokens=4)
    got = nn.generate(m, t, max_new_tokens=4, past_key_values=nn.QuantizedCache())
    assert got.shape == ref.shape and (got == ref).float().mean() > 0.8


def test_quantised_linear_modules_track_the_float_layer():
    torch.manual_seed(0)
    lin = tnn.Linear(128, 64)
    x = torch.randn(8, 128)
    ref = lin(x)
    for mode, tol in (("int8_weight_only", 0.03), ("int8_dynamic", 0.05), ("float8_weight_only", 0.12),
                      ("int4_weight_only", 0.25)):
        m = Q.quantize_(tnn.Sequential(tnn.Linear(128, 64)), mode)
        m[0].load_state_dict(m[0].state_dict())         # buffers round-trip
        q = Q.quantize_(tnn.Sequential(_copy(lin)), mode)
        err = (q(x).float() - ref).norm() / ref.norm()
        assert err < tol, (mode, float(err))
    kinds = {type(Q.quantize_(tnn.Sequential(_copy(lin)), m)[0]).__name__ for m in ("int8_dynamic", "float8_weight_only")}
    assert kinds == {"Int8DynamicLinear", "Float8Linear"}


def _copy(lin):
    import copy
    return copy.deepcopy(lin)


def test_metric_collection_and_conversion(tmp_path):
    mc = metrics.MetricCollection({"acc": metrics.Accuracy(num_classes=3), "f1": metrics.F1Score(num_classes=3, average="macro")})
    logits = torch.tensor([[2.0, 0, 0], [0, 2.0, 0], [0, 0, 2.0], [2.0, 0, 0]])
    mc.update(logits, torch.tensor([0, 1, 2, 1]))
    out = mc.compute()
    assert abs(out["acc"].item() - 0.75) < 1e-6 and 0 < out["f1"].item() < 1
    mc.reset()
    mc.update(logits, torch.tensor([0, 1, 2, 0]))
    assert mc.compute()["acc"].item() == 1.0
    # torch zip -> .mega conversion keeps values and metadata is inspectable
    src, dst = str(tmp_path / "w.pt"), str(tmp_path / "w.mega")
    state = {"a": torch.arange(6.0).view(2, 3), "b": torch.ones(4, dtype=torch.bfloat16)}
    tp.save(state, src)
    tp.serialization.convert_to_mega(src, dst)
    back = tp.load(dst)
    assert set(back) == {"a", "b"} and torch.equal(back["a"], state["a"]) and back["b"].dtype == torch.bfloat16
    assert tp.inspect_checkpoint(dst)["format"] == "mega"


def test_flop_counter_tensorboard_prefetcher_and_memory_plan(tmp_path):
    from tensorplay_b200.distributed._tools import engine_memory_plan
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine
    from tensorplay_b200.utils.data import CudaPrefetcher
    from tensorplay_b200.utils.flop_counter import FlopCounterMode
    from tensorplay_b200.utils.tensorboard import SummaryWriter
    lin = tnn.Linear(32, 16, bias=False)
    with FlopCounterMode(display=False) as fc:
        lin(torch.randn(8, 32))
    assert fc.get_total_flops() == 2 * 8 * 32 * 16
    w = SummaryWriter(str(tmp_path / "tb"))
    w.add_scalar("loss", 1.0, 0)
    w.close()
    assert any(f.startswith("events.out") for f in os.listdir(tmp_path / "tb"))
    batches = [(torch.full((2,), float(i)), {"y": torch.tensor(i)}) for i in range(3)]
    got = list(CudaPrefetcher(batches, "cpu"))
    assert len(got) == 3 and float(got[2][0][0]) == 2.0 and int(got[1][1]["y"]) == 1
    cfg = LlamaConfig.tiny(hidden_size=32, num_heads=4, num_kv_heads=2, head_dim=8, ffn_size=48, vocab_size=64, num_layers=2)
    eng = FSDPEngine(Llama(cfg), AdamWConfig())
    plan = engine_memory_plan(eng)
    n_params = sum(p.numel() for p in eng.model.parameters())
    assert plan["units"] == len(eng.units) and plan["sharded_state_bytes"] >= n_params * 16


def test_grad_scaler_with_fused_adamw_and_autocast():
    from tensorplay_b200 import amp
    torch.manual_seed(0)
    lin = tnn.Linear(8, 4)
    ref = tnn.Linear(8, 4)
    ref.load_state_dict(lin.state_dict())
    opt, ropt = optim.AdamW(lin.parameters(), lr=1e-2), torch.optim.AdamW(ref.parameters(), lr=1e-2)
    scaler = amp.GradScaler("cpu", init_scale=1024.0)
    x = torch.randn(16, 8)
    for _ in range(3):
        with amp.autocast("cpu", dtype=torch.bfloat16):
            loss = lin(x).float().pow(2).mean()
        opt.zero_grad()
        scaler.scale(loss).backward()
        scaler.step(opt)
        scaler.update()
        with amp.autocast("cpu", dtype=torch.bfloat16):
            l2 = ref(x).float().pow(2).mean()
        ropt.zero_grad()
        l2.backward()
        ropt.step()
    torch.testing.assert_close(lin.weight, ref.weight, rtol=1e-5, atol=1e-6)   # unscaled inside the step
    w0 = lin.weight.detach().clone()
    opt.zero_grad()
    scaler.scale(lin(x).pow(2).mean()).backward()
    lin.weight.grad[0, 0] = float("inf")
    scaler.step(opt)
    scaler.update()
    assert torch.equal(lin.weight, w0) and scaler.get_scale() == 512.0          # step skipped, scale halved


def test_reexported_utilities_smoke():
    from tensorplay_b200 import autograd, profiler
    from tensorplay_b200.utils.checkpoint import checkpoint_sequential
    from tensorplay_b200.utils.data import DistributedSampler, TensorDataset
    ds = TensorDataset(torch.arange(10))
    parts = [list(DistributedSampler(ds, num_replicas=2, rank=r, shuffle=False)) for r in range(2)]
    assert sorted(parts[0] + parts[1]) == list(range(10))
    seq = tnn.Sequential(tnn.Linear(4, 4), tnn.Tanh(), tnn.Linear(4, 4), tnn.Tanh())
    x = torch.randn(3, 4, requires_grad=True)
    y = checkpoint_sequential(seq, 2, x, use_reentrant=False)
    torch.testing.assert_close(y, seq(x))
    y.sum().backward()
    assert x.grad is not None
    f = lambda a: (a ** 3).sum()   # noqa: E731
    assert autograd.gradcheck(f, (torch.randn(4, dtype=torch.float64, requires_grad=True),))
    with profiler.profile(activities=[profiler.ProfilerActivity.CPU]) as prof:
        with profiler.record_function("my_region"):
            torch.randn(64, 64) @ torch.randn(64, 64)
    assert any(e.key == "my_region" for e in prof.key_averages())


def test_every_cache_kind_reproduces_cache_free_generation():
    torch.manual_seed(0)
    m = nn.DecoderLM(48, 32, 2, 4, 2)
    t = torch.randint(0, 48, (2, 5))
    ref = nn.generate(m, t, max_new_tokens=6, use_cache=False)
    for cache in (nn.DynamicCache(), nn.StaticCache(32), nn.PagedCache(block_size=4), nn.SlidingWindowCache(64)):
        out = nn.generate(m, t, max_new_tokens=6, past_key_values=cache)
        assert torch.equal(out, ref), type(cache).__name__
        assert cache.get_seq_length(0) == 10               # 5 prompt + 5 fed-back tokens
    # module-level pieces against formulas
    x = torch.randn(3, 7, 32)
    norm = nn.RMSNorm(32, eps=1e-6)
    torch.testing.assert_close(norm(x), x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * norm.weight)
    y, s = norm(x, residual=x)
    torch.testing.assert_close(s, 2 * x)
    att = nn.GroupedQueryAttention(32, 4, 2)
    full = att(x)
    torch.testing.assert_close(att(x[:, :4]), full[:, :4], rtol=1e-5, atol=1e-5)    # causal: a prefix is unchanged


def test_swap_in_optimizer_params_and_state():
    torch.manual_seed(0)
    lin = tnn.Linear(4, 2)
    opt = torch.optim.SGD(lin.parameters(), lr=0.1, momentum=0.9)
    lin(torch.randn(3, 4)).sum().backward()
    opt.step()
    own = [p.detach().clone() for p in lin.parameters()]
    copies = {n: p.detach().clone().requires_grad_() for n, p in lin.named_parameters()}
    sd = opt.state_dict()
    sd["param_groups"][0]["lr"] = 1.0
    with optim.swap_in_optimizer_params_and_state(opt, copies, sd):
        for p in copies.values():
            p.grad = torch.ones_like(p)
        opt.step()
    assert opt.param_groups[0]["lr"] == 0.1                                   # hyper-parameters restored
    for p, o in zip(lin.parameters(), own):
        assert torch.equal(p, o)                                                # the live model did not move
    assert all(not torch.equal(c, o) for c, o in zip(copies.values(), own))     # the copies did


def test_serialization_helpers_and_trace_merge(tmp_path):
    import gzip
    import json

    import torch

    import tensorplay_b200 as tp
    from tensorplay_b200 import serialization as S
    state = {"w": torch.arange(6.0).reshape(2, 3), "b": torch.ones(3, dtype=torch.bfloat16)}
    src = tmp_path / "model.safetensors"
    S.save_safetensors(state, str(src))
    out = S.convert_model(str(src))
    assert out == str(tmp_path / "model.mega") and S.sniff_format(out) == "mega"
    hdr = S.parse_mega_header(out)
    assert hdr["file_size"] == (tmp_path / "model.mega").stat().st_size
    back = S.load(out)
    assert torch.equal(back["w"], state["w"]) and back["b"].dtype == torch.bfloat16
    # a sharded directory: every shard is converted and the index follows the new names
    shard_dir = tmp_path / "sharded"
    S.save_sharded({f"layer{i}.w": torch.full((4, 4), float(i)) for i in range(4)}, str(shard_dir), max_shard_bytes=100,
                   format="safetensors")
    mega_dir = S.convert_to_mega(str(shard_dir), str(tmp_path / "as_mega"))
    files = sorted(p.name for p in (tmp_path / "as_mega").iterdir())
    assert "model.mega.index.json" in files and all(f.endswith((".mega", ".json")) for f in files)
    got = S.load_sharded(mega_dir)
    assert sorted(got) == [f"layer{i}.w" for i in range(4)] and float(got["layer3.w"][0, 0]) == 3.0
    assert S.resolve_map_location(None, "cuda:0") is None
    assert S.resolve_map_location("cpu", "cuda:0") == torch.device("cpu")
    assert S.resolve_map_location({"cuda:0": "cpu"}, "cuda:0") == torch.device("cpu")
    assert S.resolve_map_location({"cuda:1": "cpu"}, "cuda:0") == torch.device("cuda:0")
    assert S.resolve_map_location(lambda storage, loc: "cpu" if loc.startswith("cuda") else None, "cuda:3") == torch.device("cpu")
    assert (S.DEFAULT_ALIGNMENT, S.MEGA_EXTENSION, S.MEGA_INDEX_SUFFIX) == (4096, ".mega", ".mega.index.json")

    traces = []
    for rank in (1, 0):
        path = tmp_path / f"trace{rank}.json.gz"
        with gzip.open(path, "wt") as f:
            json.dump({"distributedInfo": {"rank": rank}, "traceEvents": [{"name": f"k{rank}", "pid": 7, "ts": rank}]}, f)
        traces.append(str(path))
    merged = tp.profiler.merge_distributed_traces(traces, str(tmp_path / "all.json"))
    doc = json.load(open(merged))
    assert doc["distributedInfo"]["merged_ranks"] == [1, 0]
    assert sorted(e["pid"] for e in doc["traceEvents"]) == [7, 10_000_007]
    assert tp.quantum.decode_w(tp.quantum.encode_w([1, 3, 2])) == [1, 3, 2] and tp.quantum.encode_w(4) == "4"
    import datetime
    assert isinstance(tp.distributed.default_pg_timeout, datetime.timedelta)
    from tensorplay_b200.func import vmap
    from tensorplay_b200.linalg import svd   # noqa: F401
    assert float(vmap(lambda v: v.sum())(torch.ones(2, 3))[0]) == 3.0
