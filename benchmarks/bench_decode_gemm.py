"""Few-row (decode) GEMMs: the four projections of a Llama-3-70B layer at tensor-parallel degree 8 with M = 64 and
M = 8 rows, with and without the K-split of the tiles, as microseconds per launch and GB/s of weight bytes.

    python benchmarks/bench_decode_gemm.py

Each shape runs from a CUDA graph that rotates through enough weight matrices to exceed the 126 MB L2, so every launch
streams its weights from HBM; CUDA events around 30 replays after 5 warm-ups.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.ops.gemm import enable_splitk  # noqa: E402


def timeit(fn, iters=30, warmup=5):
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


def main():
    shapes = [("qkv", 1280, 8192), ("o", 8192, 1024), ("gate_up", 7168, 8192), ("down", 8192, 3584)]
    for M in (64, 8):
        for label, split in (("one CTA per tile", False), ("tiles split along K", True)):
            enable_splitk(enable=split)
            total, cells = 0.0, []
            for name, N, K in shapes:
                ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) for _ in range(max(2, int(400e6 // (N * K * 2))))]
                x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
                out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
                i = [0]

                def f():
                    O.gemm(x, ws[i[0] % len(ws)], out=out, impl="single")
                    i[0] += 1
                f()
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(len(ws)):
                        f()
                ms = timeit(g.replay) / len(ws)
                total += ms
                cells.append(f"{name} {ms * 1e3:.1f} us ({N * K * 2 / ms / 1e6:.0f} GB/s)")
            print(f"M={M} {label:22s} sum {total * 1e3:6.1f} us | " + " | ".join(cells), flush=True)
    enable_splitk(enable=False)
    O.check_status()


if __name__ == "__main__":
    main()
