"""Per-stream timeline summary of one training step of the sharded engine on N GPUs (rank 0's view).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/profile_step_dist.py --layers 8

Prints, per CUDA stream, the busy time and the largest kernels, plus the idle time of the compute
stream inside the step: the part of the communication that is not hidden shows up there.
"""
import argparse
import json
import os
import sys
import tempfile
from collections import defaultdict

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    a = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig.llama3_8b()
    cfg.num_layers = a.layers
    model = Llama(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(seed=0)
    eng = FSDPEngine(model, AdamWConfig())
    tok = torch.randint(0, cfg.vocab_size, (1, 4096), device=dev)
    for _ in range(3):
        eng.step(tok, tok)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        eng.step(tok, tok)
    e1.record()
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / 3
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step(tok, tok)
        torch.cuda.synchronize()
    if rank == 0:
        path = os.path.join(tempfile.mkdtemp(), "trace.json")
        prof.export_chrome_trace(path)
        with open(path) as f:
            tr = json.load(f)
        ev = [e for e in tr["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
        by_stream = defaultdict(list)
        for e in ev:
            by_stream[e.get("args", {}).get("stream", -1)].append(e)
        t0 = min(e["ts"] for e in ev)
        t1 = max(e["ts"] + e["dur"] for e in ev)
        print(f"# Llama-3-8B shape, {a.layers} layers, {world} GPU(s): step {step_ms:.2f} ms (CUDA events, no profiler); "
              f"profiled span {(t1 - t0) / 1e3:.2f} ms")
        for sid, es in sorted(by_stream.items(), key=lambda kv: -sum(e["dur"] for e in kv[1])):
            es.sort(key=lambda e: e["ts"])
            busy = sum(e["dur"] for e in es)
            # union length (kernels of one stream do not overlap, but be safe)
            cur_end, union = 0, 0
            for e in es:
                s_, en = e["ts"], e["ts"] + e["dur"]
                if s_ > cur_end:
                    union += en - s_
                    cur_end = en
                elif en > cur_end:
                    union += en - cur_end
                    cur_end = en
            span = es[-1]["ts"] + es[-1]["dur"] - es[0]["ts"]
            print(f"stream {sid}: {len(es)} ops, busy {busy / 1e3:.2f} ms, first-to-last span {span / 1e3:.2f} ms, idle inside span {(span - union) / 1e3:.2f} ms")
            gaps = []
            for x, y in zip(es[:-1], es[1:]):
                g_ = y["ts"] - (x["ts"] + x["dur"])
                if g_ > 20:
                    gaps.append((g_, x["name"][:48], y["name"][:48]))
            gaps.sort(reverse=True)
            tot_gap = sum(g_[0] for g_ in gaps)
            print(f"    gaps > 20 us: {len(gaps)} totalling {tot_gap / 1e3:.2f} ms; largest:")
            for g_, x, y in gaps[:14]:
                print(f"      {g_ / 1e3:7.3f} ms  after [{x}] before [{y}]")
            agg = defaultdict(lambda: [0.0, 0])
            for e in es:
                k = e["name"][:70]
                agg[k][0] += e["dur"]
                agg[k][1] += 1
            for k, (d, c) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:8]:
                print(f"    {d / 1e3:8.3f} ms x{c:4d}  {k}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
