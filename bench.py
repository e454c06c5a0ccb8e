"""Flagship benchmark: Llama-3-8B-shape training step (fully sharded, bf16 params/activations,
fp32 AdamW state, activation checkpointing, seq 4096, micro-batch 1 per GPU), tokens/s per box.

    python bench.py --gpus 1 --steps K --warmup W
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Rank 0 prints ONE JSON line. ``value`` is device-timed (CUDA events around exactly K steps,
barrier + synchronize on both sides, max over ranks) with inputs resident on the device; ``e2e``
repeats the K steps through the public API with a pinned-host -> device copy of each step's
tokens/targets and a device -> host read of the loss inside the timed region.
``--impl reference`` is the reference arm (lexing-2026/TensorPlay installed under
baseline/_ref); it reports ``unavailable`` when that install does not exist.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "tiny", "qwen3_moe"],
                    help="llama3_8b = the headline config; qwen3_moe = the Qwen3-30B-A3B-shape MoE config with expert "
                         "parallelism over all ranks (same JSON contract, its own metric name)")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--comm", default="auto", choices=["auto", "symm", "torch"])
    ap.add_argument("--ac", default="selective", choices=["full", "selective"],
                    help="activation checkpointing per transformer block: keep the GEMM / attention outputs and "
                         "recompute only norms, RoPE and SwiGLU in backward (the default: same gradients, bit for "
                         "bit, and 12 GB of kept activations fit beside the shards), or recompute the whole block")
    ap.add_argument("--layers", type=int, default=None,
                    help="debug only: fewer layers (the JSON then names the reduced model)")
    return ap.parse_args()


def reference_arm(args):
    """Runs the unmodified reference from ``baseline/_ref`` when an install exists there; prints the
    ``unavailable`` line otherwise. The install was attempted offline (pip --no-index --no-build-isolation
    from a copy of the source tree): 565 of its 567 objects compile for sm_100 once the cuDNN-frontend and
    CUTLASS headers of this image are staged into the copy, then the build stops because
    src/distributed/bindings.cpp and src/distributed/mpi/ProcessGroupMPI.cpp include gloo headers
    unconditionally (also with gloo, MPI and the distributed package switched off in CMake) and no gloo
    source or headers exist on a machine without network."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref_dir, "tensorplay")):
        why = ("reference not installed: offline build compiles 565/567 objects for sm_100, then fails on "
               "<gloo/context.h> (src/distributed/bindings.cpp, src/distributed/mpi/ProcessGroupMPI.cpp include "
               "gloo unconditionally; no gloo headers on this image, no network)")
    else:
        sys.path.insert(0, ref_dir)
        try:
            import tensorplay  # noqa: F401
            why = ("reference imports, but no Llama-3-8B FSDP training recipe of it has been validated on this "
                   "box; not timed")
        except Exception as e:  # pragma: no cover - depends on an install that cannot be produced offline
            why = f"reference import failed: {type(e).__name__}: {str(e)[:160]}"
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                  "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples is "under load"
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_mhz_median_upper_half": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from tensorplay_b200 import _native
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.parallel import AdamWConfig, FSDPEngine
    import tensorplay_b200.ops as ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    B, T = args.micro_batch, args.seq
    opt = AdamWConfig(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    torch.manual_seed(1234)
    if args.model == "qwen3_moe":
        from tensorplay_b200.models.qwen3_moe import Qwen3MoE, Qwen3MoEConfig
        cfg = Qwen3MoEConfig.qwen3_30b_a3b(max_seq_len=T)
        name = "Qwen3-30B-A3B-shape"
        metric = "train tokens/s/box, Qwen3-30B-A3B-shape MoE expert-parallel bf16, max over ranks"
        if args.layers is not None:
            cfg.num_layers = args.layers
            name += f"-{args.layers}layers(debug)"
        model = Qwen3MoE(cfg, device=dev, dtype=torch.bfloat16)
        model.reset_parameters(seed=1234)
        # arena head-room for the expert-parallel workspace (3 row buffers of `world` x the mean load)
        ws_bytes = 3 * (B * T * cfg.top_k * world + 4096) * cfg.hidden_size * 2 + (256 << 20)
        engine = FSDPEngine(model, opt, comm=args.comm,
                            activation_checkpointing=True if args.ac == "full" else "selective",
                            symm_extra_bytes=ws_bytes)
        # drop-less for any routing: one rank may receive every token of the box
        model.attach_workspace(B * T, capacity_factor=float(world))
        parallelism = f"ep{world} experts, fsdp{world} attention/embeddings"
        ac_text = ("per block, full recompute" if args.ac == "full" else
                   "per block, selective: dense projection and attention outputs kept, norms / RoPE / router top-k / "
                   "expert FFN recomputed")
    else:
        if args.model == "tiny":
            cfg = LlamaConfig.tiny(max_seq_len=T)
            name = "llama-tiny"
        else:
            cfg = LlamaConfig.llama3_8b(max_seq_len=T)
            name = "Llama-3-8B-shape"
        metric = "train tokens/s/box, Llama-3-8B-shape FSDP bf16, max over ranks"
        if args.layers is not None:
            cfg.num_layers = args.layers
            name += f"-{args.layers}layers(debug)"
        model = Llama(cfg, device=dev, dtype=torch.bfloat16)
        model.reset_parameters(seed=1234)
        engine = FSDPEngine(model, opt, comm=args.comm,
                            activation_checkpointing=True if args.ac == "full" else "selective")
        parallelism = f"fsdp{world}" if world > 1 else "single-gpu (fsdp1)"
        ac_text = ("per block, full recompute" if args.ac == "full" else
                   "per block, selective: GEMM and attention outputs kept, norms / RoPE / SwiGLU recomputed")
    gen = torch.Generator(device="cpu")
    gen.manual_seed(100 + rank)
    n_batches = max(args.steps, 1)
    host_tok = [torch.randint(0, cfg.vocab_size, (B, T), generator=gen).pin_memory() for _ in range(n_batches)]
    host_tgt = [torch.randint(0, cfg.vocab_size, (B, T), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_tok = [t.to(dev) for t in host_tok]
    dev_tgt = [t.to(dev) for t in host_tgt]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    losses = []
    for i in range(args.warmup):
        loss = engine.step(dev_tok[i % n_batches], dev_tgt[i % n_batches])
    barrier()
    ops.check_status()

    # ---------------- device-timed region: exactly K steps
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _native.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = engine.step(dev_tok[i % n_batches], dev_tgt[i % n_batches])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = _native.launch_count - launches0
    clocks = sampler.stop() if rank == 0 else None
    last_loss = float(loss.item())
    ops.check_status()

    # ---------------- end-to-end region through the public API: H2D inputs, D2H loss each step
    loss_host = torch.empty(1, dtype=torch.float32).pin_memory()
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        tok = host_tok[i % n_batches].to(dev, non_blocking=True)
        tgt = host_tgt[i % n_batches].to(dev, non_blocking=True)
        loss = engine.step(tok, tgt)
        loss_host.copy_(loss.reshape(1), non_blocking=False)
        losses.append(float(loss_host[0]))
    barrier()
    e2e_s = time.perf_counter() - t0

    t = torch.tensor([ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_ms_max = float(t[0]), float(t[1])
    tokens_per_step = world * B * T
    value = tokens_per_step * args.steps / (ms_max / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms_max / 1e3)
    if rank == 0:
        flops = (cfg.flops_per_token(T, backward=True, recompute=False) * tokens_per_step * args.steps
                 if hasattr(cfg, "flops_per_token") else 0.0)
        out = {
            "metric": metric,
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_max / args.steps, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform random token ids, random-init N(0, 0.02) weights)",
            "config": {"model": name, "global_batch": world * B, "seq_len": T,
                       "parallelism": parallelism,
                       "activation_checkpointing": ac_text, "optimizer": "AdamW fp32 state + fp32 master",
                       "comm": engine.comm_kind,
                       "l2": "per-step working set (parameters + optimizer state, >100 GB/box) "
                             "exceeds the 126 MB L2; no explicit flush"},
            "model_tflops_per_gpu": round(flops / (ms_max / 1e3) / world / 1e12, 1),
            "loss": round(last_loss, 4),
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * B * T * 8 * world, "d2h_bytes_per_step": 4 * world,
                    "ms_per_step": round(e2e_ms_max / args.steps, 3)},
            "gpu_launches": launches,
            "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
