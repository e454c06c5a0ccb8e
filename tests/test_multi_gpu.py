"""Multi-GPU tests (need >= 2 B200s): run as torchrun children, one rank per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_workers(script, nproc, timeout=600, extra_env=None):
    env = dict(os.environ)
    env.setdefault("TPB_SYMM_CANARY", "1")  # guard bytes behind every symmetric allocation, checked at close / exit
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "workers", script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    return r


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fsdp_symm_matches_nccl_and_dense():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("fsdp_symm_worker.py", n)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_symmetric_collectives_match_nccl_bit_for_bit():
    """All-gather (pull, copy engines, multicast push), reduce-scatter and all-reduce (multimem and
    plain peer loads) against NCCL on integer patterns, on every GPU of the box."""
    r = _run_workers("symm_collectives_worker.py", _ngpu())
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fsdp_multicast_transport():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("fsdp_symm_worker.py", n, extra_env={"TPB_COMM_TRANSPORT": "mc"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tp_fused_ag_gemm_and_gemm_rs():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("tp_fused_worker.py", n)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_moe_expert_parallel_dispatch_combine():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("moe_ep_worker.py", n)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tp_llama_prefill_and_decode():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("tp_llama_worker.py", n)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_ring_attention_and_clipped_step():
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("cp_worker.py", n)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fsdp_symm_pull_kernel_transport():
    """Same check with the SM pull kernels instead of the copy engines."""
    n = 2 if _ngpu() < 4 else 4
    r = _run_workers("fsdp_symm_worker.py", n, extra_env={"TPB_COMM_TRANSPORT": "sm"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "RESULT" in r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("tp,pp", [(2, 1), (1, 2)])
def test_tensor_parallel_and_pipeline_training_on_two_gpus(tp, pp):
    """Several tensor-parallel blocks trained through the fused linears (tp2), and two pipeline
    stages over NCCL point-to-point (pp2): the step runs and the loss is that of a random model."""
    import json
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "benchmarks", "bench_llama_3d.py"), "--tp", str(tp), "--pp", str(pp), "--layers", "8",
           "--microbatches", "4", "--steps", "2", "--warmup", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert 10.0 < line["loss"] < 13.5, line   # ln(128256) = 11.76


@pytest.mark.skipif(_ngpu() < 4, reason="needs 4 GPUs")
def test_composed_tp_pp_layout_trains():
    """TP2 x PP2 of the composed-layout benchmark on a short Llama-shaped model: runs, loss near ln(V)."""
    import json
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "benchmarks", "bench_llama_3d.py"), "--layers", "8", "--microbatches", "4",
           "--steps", "2", "--warmup", "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert 10.0 < line["loss"] < 13.5, line   # ln(128256) = 11.76
