"""Kernel-time table of one training step of the sharded engine (torch.profiler, CUDA activities).

    python benchmarks/profile_step.py --layers 4 [--ac full|selective] [--out profiles/step_kernels.txt]
    python benchmarks/profile_step.py --model qwen3_moe --layers 4 --experts 16
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/profile_step.py \
        --model qwen3_moe --layers 4 --experts 32          # expert parallel over the ranks; rank 0 reports
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
    ap.add_argument("--model", default="llama", choices=["llama", "qwen3_moe"])
    ap.add_argument("--experts", type=int, default=128)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    if a.model == "llama":
        cfg = LlamaConfig.llama3_8b()
        cfg.num_layers = a.layers
        model = Llama(cfg, device=dev, dtype=torch.bfloat16)
        model.reset_parameters(seed=0)
        eng = FSDPEngine(model, AdamWConfig(), activation_checkpointing=True if a.ac == "full" else "selective")
        shape = f"Llama-3-8B shape with {a.layers} layers"
    else:
        from tensorplay_b200.models.qwen3_moe import Qwen3MoE, Qwen3MoEConfig
        cfg = Qwen3MoEConfig.qwen3_30b_a3b(num_experts=a.experts)
        cfg.num_layers = a.layers
        model = Qwen3MoE(cfg, device=dev, dtype=torch.bfloat16)
        model.reset_parameters(seed=0)
        ws_bytes = 3 * (4096 * cfg.top_k * world + 4096) * cfg.hidden_size * 2 + (256 << 20)
        a.ac = "full"
        eng = FSDPEngine(model, AdamWConfig(), activation_checkpointing=True, symm_extra_bytes=ws_bytes)
        model.attach_workspace(4096, capacity_factor=float(world))
        shape = f"Qwen3-30B-A3B shape with {a.layers} layers, {a.experts} experts, EP={world}"
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
    if rank != 0:
        return
    lines = [f"# kernel time per step, {shape}, seq 4096, {world} GPU(s), "
             f"activation checkpointing {a.ac} (torch.profiler)",
             f"# total device kernel time per step: {total / 1e3:.2f} ms; CUDA-event step time without "
             f"the profiler: {step_ms:.2f} ms (kernels on side streams overlap, gaps are idle time)"]
    for t, c, k in rows[:45]:
        lines.append(f"{t / 1e3:9.3f} ms {100 * t / total:5.1f}%  x{c:4d}  {k[:90]}")
    text = "\n".join(lines)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
