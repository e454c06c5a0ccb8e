"""GPT-2-small-shape training (12 layers, d=768, 12 heads, vocab 50257, context 1024, micro-batch
16 per GPU, bf16 parameters with fp32 master + AdamW state) under DDP (25 MB buckets; fused
all-reduce + AdamW over peer memory, or NCCL all-reduce + fused AdamW) and under the sharded
engine (FSDP). Tokens/s per box, CUDA-event timed, max over ranks.

    python benchmarks/bench_gpt2.py --mode ddp|ddp-nccl|fsdp  [torchrun for N > 1]
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP  # noqa: E402
from tensorplay_b200.models.gpt2 import GPT2, GPT2Config  # noqa: E402
from tensorplay_b200.optim import AdamW  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="ddp", choices=["ddp", "ddp-nccl", "fsdp"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--micro-batch", type=int, default=16)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = GPT2Config.small()
    model = GPT2(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(seed=0)
    ocfg = AdamWConfig(lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    B, T = a.micro_batch, cfg.n_ctx
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(dev)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(dev)
    if a.mode == "fsdp":
        eng = FSDPEngine(model, ocfg, activation_checkpointing=False)
        step = lambda: eng.step(tok, tgt)
    elif a.mode == "ddp" and world > 1:
        ddp = DDP(model, bucket_cap_mb=25, fused_adamw=ocfg)

        def step():
            loss = ddp(tok, tgt)
            loss.backward()
            ddp.finish_step()
            return loss
    else:
        ddp = DDP(model, bucket_cap_mb=25, comm="torch")
        opt = AdamW(model.parameters(), lr=ocfg.lr, betas=ocfg.betas, eps=ocfg.eps, weight_decay=ocfg.weight_decay)

        def step():
            loss = ddp(tok, tgt)
            loss.backward()
            ddp.synchronize()
            opt.step()
            for b in ddp.buckets:
                b.flat_grad.zero_()
            return loss
    for _ in range(a.warmup):
        loss = step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    O.check_status()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t[0]) / a.steps
        print(json.dumps({"config": f"GPT-2-small-shape {a.mode}, micro-batch {B} x {T} per GPU, bf16 + fp32 master",
                          "n_gpus": world, "tokens_per_s": round(world * B * T / (ms / 1e3), 1),
                          "ms_per_step": round(ms, 3), "loss": round(float(loss.detach()), 4), "data": "synthetic"}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
