"""Quantised kernels on one B200: int8 tensor-core GEMM (A8W8) against the bf16 GEMM of the same
shape, and the weight-only GEMV (W8A16 / W4A16) against its weight-streaming roofline.

    python benchmarks/bench_quant.py                      # all numbers
    python benchmarks/bench_quant.py --profile-gemv 8     # small case for a profiler capture (also 4)
CUDA events, 3 warm-ups; every operand set is larger than the 126 MB L2 or rotated so that weights
come from HBM.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.ops.quant import gemv_config  # noqa: E402


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


def profile_gemv(bits: int) -> None:
    """A few eager calls of the default GEMV kernel over four weight sets (0.5-0.9 GB on the device):
    the case to run under a profiler (``ncu --clock-control none -k regex:wq_gemv_mma -c 2``, on this small case only)."""
    dev = "cuda"
    N, K, M, group = 28672, 8192, 8, (0 if bits == 8 else 128)
    x = torch.randn(M, K, device=dev).bfloat16()
    ws = []
    for _ in range(4):
        w = torch.randn(N, K, device=dev)
        ws.append(O.quantize_weight_int8(w) + (None,) if bits == 8 else O.quantize_weight_int4(w, group))
        del w
    for i in range(6):
        q, s, z = ws[i % 4]
        O.weight_only_linear(x, q, s, z, None, bits, group)
    torch.cuda.synchronize()
    O.check_status()
    print(json.dumps({"profiled": f"W{bits}A16 GEMV", "calls": 6}), flush=True)


def main():
    dev = "cuda"
    if "--profile-gemv" in sys.argv:
        return profile_gemv(int(sys.argv[sys.argv.index("--profile-gemv") + 1]))
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f).get("hbm_gbs", 6650.0))
    except Exception:
        hbm = 6650.0
    out = []
    for M, N, K in ((8192, 8192, 8192), (4096, 28672, 4096)):
        a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
        sa, sw = torch.rand(M, device=dev), torch.rand(N, device=dev)
        ab, wb = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
        t8 = timeit(lambda: O.int8_gemm(a, w, sa, sw))
        t16 = timeit(lambda: O.gemm(ab, wb))
        out.append({"kernel": "int8_gemm (tcgen05 kind::i8, scaled bf16 out)", "shape": [M, N, K], "ms": round(t8, 4),
                    "tops": round(2.0 * M * N * K / t8 / 1e9, 1), "bf16_gemm_ms": round(t16, 4),
                    "bf16_tflops": round(2.0 * M * N * K / t16 / 1e9, 1)})
    # decode GEMV: 8 rotating weight matrices (1.9 GB of int8) so that every call streams from HBM
    N, K, M = 28672, 8192, 8
    x = torch.randn(M, K, device=dev).bfloat16()
    for bits, group in ((8, 0), (4, 128)):
        ws = []
        for _ in range(8):
            w = torch.randn(N, K, device=dev)
            ws.append(O.quantize_weight_int8(w) + (None,) if bits == 8 else O.quantize_weight_int4(w, group))
            del w
        i = [0]

        def run():
            q, s, z = ws[i[0] % 8]
            i[0] += 1
            O.weight_only_linear(x, q, s, z, None, bits, group)

        wbytes = N * K * bits // 8
        for label, tiles, simt, ver, fold in (
                ("warp-MMA, chosen tiles", 0, False, 1, True), ("warp-MMA, 1 tile per CTA", 1, False, 1, True),
                ("warp-MMA, 2 tiles per CTA", 2, False, 1, True),
                ("warp-MMA second version, scaling per weight", 0, False, 2, False),
                ("warp-MMA second version (4 bits: scaling per 128-k chunk), chosen tiles", 0, False, 2, True),
                ("warp-MMA second version (4 bits: scaling per 128-k chunk), 2 tiles per CTA", 2, False, 2, True),
                ("CUDA-core FMA kernel", 0, True, 1, True)):
            gemv_config(tiles, simt, ver, fold)
            # sixteen calls (two passes over the eight weight sets) replayed from a CUDA graph: the
            # kernel is shorter than the host-side cost of one call, so eager timing would measure Python
            run()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(16):
                    run()
            t = timeit(graph.replay, iters=10) / 16
            out.append({"kernel": f"W{bits}A16 GEMV ({label})", "shape": [M, N, K], "group": group,
                        "ms": round(t, 4), "weight_gbs": round(wbytes / t / 1e6, 1),
                        "fraction_of_measured_hbm": round(wbytes / t / 1e6 / hbm, 3)})
        gemv_config(0, False, 2)
    O.check_status()
    for o in out:
        print(json.dumps(o), flush=True)


if __name__ == "__main__":
    main()
