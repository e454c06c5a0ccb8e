"""Kernel-time table of one training step of the sharded engine (torch.profiler, CUDA activities).

    python benchmarks/profile_step.py --layers 4 [--ac full|selective] [--out profiles/step_kernels.txt]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--out", default=None)
    ap.add_argument("--ac", default="selective", choices=["full", "selective"])
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    cfg = LlamaConfig.llama3_8b()
    cfg.num_layers = a.layers
    model = Llama(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(seed=0)
    eng = FSDPEngine(model, AdamWConfig(), activation_checkpointing=True if a.ac == "full" else "selective")
    tok = torch.randint(0, cfg.vocab_size, (1, 4096), device=dev)
    for _ in range(3):
        eng.step(tok, tok)
    torch.cuda.synchronize()
    # device-timed step without the profiler, to compare with the sum of kernel times (idle gaps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        eng.step(tok, tok)
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / 3
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(2):
            eng.step(tok, tok)
        torch.cuda.synchronize()
    rows = []
    for e in prof.key_averages():
        if e.device_time_total > 0:
            rows.append((e.device_time_total / 2, e.count // 2, e.key))
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    lines = [f"# kernel time per step, Llama-3-8B shape with {a.layers} layers, seq 4096, 1 GPU, "
             f"activation checkpointing {a.ac} (torch.profiler)",
             f"# total device kernel time per step: {total / 1e3:.2f} ms; CUDA-event step time without "
             f"the profiler: {step_ms:.2f} ms (kernels on side streams overlap, gaps are idle time)"]
    for t, c, k in rows[:30]:
        lines.append(f"{t / 1e3:9.3f} ms {100 * t / total:5.1f}%  x{c:4d}  {k[:90]}")
    text = "\n".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
