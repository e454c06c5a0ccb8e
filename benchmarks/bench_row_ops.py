"""Device-timed bandwidth of the memory-bound kernels (RMSNorm, LayerNorm, RoPE, SwiGLU, GELU,
cross-entropy, fused AdamW) on Llama-3-8B-sized rows, forward and backward, as GB/s of algorithmic
bytes (every tensor read or written once) and as a fraction of the measured copy bandwidth.

    python benchmarks/bench_row_ops.py [--only NAME] [--iters N]

Inputs are larger than the 126 MB L2 (or rotate through several buffers that together are), CUDA
events on the launching stream, 5 warm-up calls. ``--only NAME --iters 2`` gives a short run of one
kernel for a profiler capture.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402

DEV = "cuda"
BF = torch.bfloat16


def peak_gbs():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timeit(fn, iters, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def cases():
    rows, H, I, V = 65536, 4096, 14336, 128256
    out = []

    # ---- RMSNorm (with and without the fused residual add)
    x = torch.randn(rows, H, device=DEV, dtype=BF)
    res = torch.randn(rows, H, device=DEV, dtype=BF)
    w = torch.ones(H, device=DEV, dtype=BF)
    out.append(("rmsnorm_fwd", lambda: O.rms_norm(x, w), 2 * x.numel() * 2))
    out.append(("rmsnorm_residual_fwd", lambda: O.rms_norm(x, w, residual=res), 4 * x.numel() * 2))
    xg = x.clone().requires_grad_(True)
    wg = w.clone().requires_grad_(True)
    y = O.rms_norm(xg, wg)
    dy = torch.randn_like(y)
    out.append(("rmsnorm_bwd", lambda: torch.autograd.grad(y, (xg, wg), dy, retain_graph=True), 3 * x.numel() * 2))

    # ---- LayerNorm
    b = torch.zeros(H, device=DEV, dtype=BF)
    out.append(("layernorm_fwd", lambda: O.layer_norm(x, w, b), 2 * x.numel() * 2))
    bg = b.clone().requires_grad_(True)
    yl = O.layer_norm(xg, wg, bg)
    out.append(("layernorm_bwd", lambda: torch.autograd.grad(yl, (xg, wg, bg), dy, retain_graph=True), 3 * x.numel() * 2))

    # ---- RoPE on q of [B, T, heads, D] (in place: one read, one write)
    q = torch.randn(4, 4096, 32, 128, device=DEV, dtype=BF)
    cos, sin = O.rope_tables(4096, 128, theta=500000.0, device=DEV)
    out.append(("rope_inplace", lambda: O.apply_rope(q, cos, sin, inplace=True), 2 * q.numel() * 2))
    # the training path: q and k heads rotated out of the packed QKV projection into a fresh buffer
    packed = torch.randn(4, 4096, 48, 128, device=DEV, dtype=BF)
    qk_src = packed[:, :, :40]
    out.append(("rope_from_packed_qkv", lambda: O.apply_rope(qk_src, cos, sin), 2 * qk_src.numel() * 2))

    # ---- SwiGLU / GELU
    rows = 16384
    gu = torch.randn(rows, 2 * I, device=DEV, dtype=BF)
    out.append(("swiglu_packed_fwd", lambda: O.swiglu_packed(gu), 3 * rows * I * 2))
    gug = gu.clone().requires_grad_(True)
    ys = O.swiglu_packed(gug)
    dys = torch.randn_like(ys)
    out.append(("swiglu_packed_bwd", lambda: torch.autograd.grad(ys, gug, dys, retain_graph=True), 5 * rows * I * 2))
    xe = torch.randn(rows, I, device=DEV, dtype=BF)
    out.append(("gelu_fwd", lambda: O.gelu(xe), 2 * xe.numel() * 2))

    # ---- cross-entropy over the Llama-3 vocabulary (forward reads the logits once; backward rewrites them)
    T = 4096
    logits = torch.randn(T, V, device=DEV, dtype=BF)
    tgt = torch.randint(0, V, (T,), device=DEV)
    out.append(("cross_entropy_fwd", lambda: O.cross_entropy(logits, tgt), logits.numel() * 2))

    def ce_fwd_bwd():
        lg = logits.detach().requires_grad_(True)
        O.cross_entropy(lg, tgt).backward()
    out.append(("cross_entropy_fwd_bwd", ce_fwd_bwd, 3 * logits.numel() * 2))

    # ---- fused AdamW on a 436 MB-parameter unit: fp32 master + two moments read and written, bf16 gradient
    # read, bf16 model copy written
    n = 218 * 1024 * 1024
    master = torch.randn(n, device=DEV)
    m1 = torch.zeros(n, device=DEV)
    m2 = torch.zeros(n, device=DEV)
    grad = torch.randn(n, device=DEV, dtype=BF)
    model = torch.empty(n, device=DEV, dtype=BF)
    step = [0]

    def adamw():
        step[0] += 1
        O.adamw_flat_(master, m1, m2, grad, model, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                      step=step[0])
    out.append(("adamw_flat", adamw, n * (3 * 4 * 2 + 2 + 2)))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=20)
    a = ap.parse_args()
    peak, how = peak_gbs()
    for name, fn, nbytes in cases():
        if a.only and a.only != name:
            continue
        ms = timeit(fn, a.iters, warmup=5 if a.iters > 2 else 1)
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "ms": round(ms, 4), "algorithmic_GB": round(nbytes / 1e9, 3),
                          "GBps": round(gbs, 1), f"frac_of_{how}_copy_bw": round(gbs / peak, 3)}), flush=True)
    O.check_status()


if __name__ == "__main__":
    main()
