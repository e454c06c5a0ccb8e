"""Fused multi-step LIF neuron on one B200: neuron-steps ("spikes") per second, forward only and
forward + backward, against the per-step module loop. CUDA events, 3 warm-ups; the [T, N] tensors
(1 GiB in fp32) are far larger than the 126 MB L2.

    python benchmarks/bench_snn.py
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200 import snn  # noqa: E402


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    dev = torch.device("cuda")
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f).get("hbm_gbs", 6650.0))
    except Exception:
        hbm = 6650.0
    T, N = 16, 16 * 1024 * 1024
    lif = snn.LIF(tau=2.0)
    for dtype, eb in ((torch.float32, 4), (torch.bfloat16, 2)):
        x = torch.randn(T, N, device=dev).to(dtype)
        t_f = timeit(lambda: snn.multi_step_lif(x))
        xg = x.clone().requires_grad_()
        gy = torch.ones_like(x)

        def fb():
            xg.grad = None
            lif(xg).backward(gy)
        t_fb = timeit(fb)
        steps = T * N
        print(json.dumps({"kernel": "fused multi-step LIF", "dtype": str(dtype), "shape": [T, N],
                          "fwd_ms": round(t_f, 4), "fwd_gspikes_per_s": round(steps / t_f / 1e6, 1),
                          "fwd_fraction_of_measured_hbm": round(steps * 2 * eb / t_f / 1e6 / hbm, 3),
                          "fwd_bwd_ms": round(t_fb, 4), "fwd_bwd_gspikes_per_s": round(steps / t_fb / 1e6, 1),
                          "fwd_bwd_fraction_of_measured_hbm": round(steps * (4 * eb + 8) / t_fb / 1e6 / hbm, 3),
                          "reference_published_gspikes_per_s": 31.0}), flush=True)
    # the per-step module loop on a smaller problem (same op, T launches of several kernels each)
    xs = torch.randn(T, 1024 * 1024, device=dev)
    cell = snn.LIFCell(tau=2.0)

    def loop():
        v = None
        for t in range(T):
            _, v = cell(xs[t], v)
    t_loop = timeit(loop)
    print(json.dumps({"kernel": "per-step LIFCell loop (torch ops)", "shape": [T, 1024 * 1024],
                      "fwd_ms": round(t_loop, 4), "fwd_gspikes_per_s": round(T * 1024 * 1024 / t_loop / 1e6, 1)}),
          flush=True)


if __name__ == "__main__":
    main()
