"""Device-timed throughput of the tcgen05 GEMM against torch.matmul (cuBLAS) on the
Llama-3-8B layer shapes. Prints one JSON line per shape; TFLOP/s from CUDA events."""
import json
import sys
import os

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.ops._common import lib as _lib  # noqa: E402


def timeit(fn, iters=20, warmup=5):
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
    shapes = [(4096, 6144, 4096), (4096, 4096, 4096), (4096, 28672, 4096), (4096, 4096, 14336),
              (4096, 128256, 4096), (8192, 8192, 8192)]
    if "--small" in sys.argv:
        shapes = [(4096, 4096, 4096)]
    if "--splitk" in sys.argv:
        from tensorplay_b200.ops.gemm import enable_splitk
        enable_splitk()
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        at, bt = a.t().contiguous(), b.t().contiguous()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        res = {"M": M, "N": N, "K": K}
        fl = 2.0 * M * N * K
        for name, fn in [
            ("tn", lambda: O.gemm(a, b, out=out)),
            ("tn_single", lambda: O.gemm(a, b, out=out, impl="single")),
            ("tn_pair", lambda: O.gemm(a, b, out=out, impl="pair")),
            ("nn_bmn_pair", lambda: O.gemm(a, bt, b_mn=True, out=out, impl="pair")),
            ("amn_bmn_pair", lambda: O.gemm(at, bt, a_mn=True, b_mn=True, out=out, impl="pair")),
            ("nn_bmn", lambda: O.gemm(a, bt, b_mn=True, out=out)),
            ("amn_bmn", lambda: O.gemm(at, bt, a_mn=True, b_mn=True, out=out)),
            ("cublas", lambda: torch.matmul(a, b.t(), out=out)),
        ]:
            ms = timeit(fn)
            res[name + "_tflops"] = round(fl / ms / 1e9, 1)
        O.check_status()
        res["resident_pairs"] = _lib().tpb_gemm_pair_resident()
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
