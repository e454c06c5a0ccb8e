"""Device-timed flash attention forward / backward on the Llama-3-8B shape
(32 q heads / 8 kv heads, head_dim 128, seq 4096, causal). One JSON line."""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.ops.attention import flash_attention  # noqa: E402


def timeit(fn, iters=10, warmup=3):
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
    B, T, Hq, Hkv, D = 2, 4096, 32, 8, 128
    if "--small" in sys.argv:
        B = 1
    q = torch.randn(B, T, Hq, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    fl_fwd = 4.0 * B * Hq * T * T * D / 2  # causal
    sweep = {}
    if "--sweep" in sys.argv:
        # share of the exponentials on the FMA pipe (n of every 4 column pairs)
        from tensorplay_b200 import _native
        for n in (0, 1, 2):
            _native.kernels().tpb_flash_fwd_config(n)
            sweep[f"fwd_ms_poly{n}"] = round(timeit(lambda: flash_attention(q, k, v, causal=True)), 4)
        _native.kernels().tpb_flash_fwd_config(1)
    ms_f = timeit(lambda: flash_attention(q, k, v, causal=True))
    o = flash_attention(q, k, v, causal=True)
    g = torch.randn_like(o)
    ms_b = timeit(lambda: torch.autograd.grad(o, (q, k, v), g, retain_graph=True))
    O.check_status()
    res = {"B": B, "T": T, "Hq": Hq, "Hkv": Hkv, "D": D, "fwd_ms": round(ms_f, 3),
           "fwd_tflops": round(fl_fwd / ms_f / 1e9, 1), "bwd_ms": round(ms_b, 3),
           "bwd_tflops": round(2.5 * fl_fwd / ms_b / 1e9, 1)}
    qq, kk, vv = (t.detach().transpose(1, 2) for t in (q, k, v))
    ms_ref = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(
        qq, kk, vv, is_causal=True, enable_gqa=True))
    res["torch_sdpa_fwd_tflops"] = round(fl_fwd / ms_ref / 1e9, 1)
    res.update(sweep)
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
