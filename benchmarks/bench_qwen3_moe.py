"""Qwen3-30B-A3B-shape MoE training with expert parallelism = world size (48 layers, hidden 2048,
32/4 heads, 128 experts of 768, top-8, seq 4096, micro-batch 1 per GPU, bf16): experts sharded over
the ranks through the peer-memory dispatch/combine + grouped tcgen05 GEMM, everything else sharded by
the training engine. Tokens/s per box, CUDA events, max over ranks.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_qwen3_moe.py
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.qwen3_moe import Qwen3MoE, Qwen3MoEConfig  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--ac", default="selective", choices=["full", "selective"],
                    help="per-block activation checkpointing: recompute everything, or keep the outputs of the dense "
                         "projections and of the attention (92 MB per layer) and recompute the rest")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = Qwen3MoEConfig.qwen3_30b_a3b(max_seq_len=a.seq, num_experts=a.experts)
    cfg.num_layers = a.layers
    model = Qwen3MoE(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(seed=0)
    # arena head-room for the expert-parallel workspace (3 row buffers of `world` x the mean load)
    ws_bytes = 3 * (a.seq * cfg.top_k * world + 4096) * cfg.hidden_size * 2 + (256 << 20)
    eng = FSDPEngine(model, AdamWConfig(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1),
                     activation_checkpointing=True if a.ac == "full" else "selective", symm_extra_bytes=ws_bytes)
    # drop-less for any routing: one rank may receive every token of the box (a random-init router
    # over 48 layers concentrates tokens on few experts, which shows up as load imbalance below)
    ws = model.attach_workspace(a.seq, capacity_factor=float(world))
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, cfg.vocab_size, (1, a.seq), generator=g).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (1, a.seq), generator=g).to(dev)
    for _ in range(a.warmup):
        loss = eng.step(tok, tgt)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    O.check_status()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for _ in range(a.steps):
        loss = eng.step(tok, tgt)
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    O.check_status()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    rows = ws.last_recv_rows.double().reshape(1) if getattr(ws, "last_recv_rows", None) is not None else t.new_zeros(1)
    rows_max = rows.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows)
    if rank == 0:
        ms = float(t[0]) / a.steps
        print(json.dumps({"config": f"Qwen3-30B-A3B-shape MoE ({a.layers} layers, {a.experts} experts, top-8), EP={world}, seq {a.seq}, bf16",
                          "n_gpus": world, "tokens_per_s": round(world * a.seq / (ms / 1e3), 1),
                          "ms_per_step": round(ms, 3), "loss": round(float(loss), 4), "data": "synthetic",
                          "activation_checkpointing": a.ac,
                          "expert_load_max_over_mean_last_layer": round(float(rows_max) * world / max(float(rows), 1.0), 2)}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
