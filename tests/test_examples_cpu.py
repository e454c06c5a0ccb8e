"""The user-facing examples run end to end on CPU with tiny settings."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable] + args, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


def test_train_example_saves_and_resumes(tmp_path):
    d = str(tmp_path / "ck")
    out = _run(["examples/train_llama_fsdp.py", "--preset", "tiny", "--steps", "6", "--seq", "32", "--log-every", "3",
                "--save", d])
    assert "step 6: loss" in out and os.path.exists(os.path.join(d, "engine.json"))
    out = _run(["examples/train_llama_fsdp.py", "--preset", "tiny", "--steps", "3", "--seq", "32", "--log-every", "3",
                "--resume", d])
    assert "step 9: loss" in out


def test_train_example_reads_a_token_file(tmp_path):
    import numpy as np
    p = tmp_path / "tok.bin"
    (np.arange(4000) % 97).astype(np.int32).tofile(p)
    out = _run(["examples/train_llama_fsdp.py", "--preset", "tiny", "--steps", "4", "--seq", "32", "--log-every", "2",
                "--data", str(p)])
    assert "step 4: loss" in out


def test_generate_example_cache_kinds():
    for kind in ("dynamic", "static", "paged"):
        out = _run(["examples/generate.py", "--new-tokens", "6", "--cache", kind])
        assert "greedy with and without cache agree: True" in out, out


def test_composed_layout_benchmark_runs_on_gloo_ranks():
    """TP2 x PP2 x FSDP1 of the composed-layout benchmark script on four CPU ranks."""
    import json
    from tests.distutil import free_port
    out = _run(["-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr", "127.0.0.1",
                "--master-port", str(free_port()), "benchmarks/bench_llama_3d.py", "--cpu", "--layers", "2",
                "--seq", "16", "--microbatches", "4", "--steps", "2", "--warmup", "1"])
    line = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
    assert line["config"]["parallelism"].startswith("tp2 x pp2") and line["n_gpus"] == 4
    assert 3.0 < line["loss"] < 6.0   # ln(128) = 4.85 at random init


def test_quantize_example_recipes():
    out = _run(["examples/quantize_model.py", "--steps", "60"])
    lines = {l.split(": perplexity")[0]: l for l in out.splitlines() if ": perplexity" in l}
    assert {"bf16/fp32 reference", "int8 weight-only", "int4 weight-only (g128)", "int4 AWQ (g128)", "2:4 pruned"} <= set(lines)
    ppl = lambda k: float(lines[k].split("perplexity")[1].split()[0])   # noqa: E731
    assert abs(ppl("int8 weight-only") - ppl("bf16/fp32 reference")) < 0.05 * ppl("bf16/fp32 reference")


def test_decoder_lm_cache_equals_recompute():
    import torch
    from tensorplay_b200 import nn
    torch.manual_seed(0)
    m = nn.DecoderLM(50, 32, 2, 4, 2, tie_embeddings=True)
    assert m.lm_head.weight is m.embed.weight
    t = torch.randint(0, 50, (2, 6))
    assert torch.equal(nn.generate(m, t, max_new_tokens=5, use_cache=True),
                       nn.generate(m, t, max_new_tokens=5, use_cache=False))
    loss = m(t[:, :-1], t[:, 1:])
    loss.backward()
    assert m.embed.weight.grad is not None


def test_uneven_inputs_example_ends_with_equal_parameters():
    out = _run(["-m", "tensorplay_b200.distributed.run", "--nproc-per-node", "2", "examples/train_ddp_uneven.py",
                "--device", "cpu", "--batches", "3"])
    assert out.count("parameters equal to rank 0: True") == 2 and "rank 1: 4 batches" in out


def test_interpretability_example_runs():
    out = _run(["examples/interpret_llm.py", "--steps", "60"])
    assert "logit lens" in out and "attribution graph with" in out and "sparse autoencoder" in out

