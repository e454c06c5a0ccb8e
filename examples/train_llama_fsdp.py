"""Train a Llama-shape model with the sharded engine (1 process per GPU, or CPU ranks over gloo).

    python examples/train_llama_fsdp.py --preset tiny --steps 20                      # one process
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/train_llama_fsdp.py --preset 8b --steps 100 --save ckpt/            # one 8-GPU box

Synthetic token stream by default; ``--data tokens.bin`` (int32, flat) reads a tokenised corpus.
Checkpoints are sharded (one ``.mega`` file per rank) and reshard on load (``--resume``).
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def batches(args, cfg, rank, world, device):
    """Synthetic tokens, or ``--data``: a flat int32 token file read by the native loader (worker
    threads fill pinned batches ahead of the step; every rank gets its own share of each epoch)."""
    if args.data:
        from tensorplay_b200.utils.data import TokenFileLoader
        loader = TokenFileLoader(args.data, args.seq, args.micro_batch, dtype=torch.int32, rank=rank, world=world,
                                 seed=1234)
        while True:
            tok, tgt, _ = loader.next_batch()
            yield tok.to(device, non_blocking=True), tgt.to(device, non_blocking=True)
    g = torch.Generator().manual_seed(1234 + rank)
    while True:
        tok = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq + 1), generator=g)
        tok = tok.pin_memory() if device.type == "cuda" else tok
        tok = tok.to(device, non_blocking=True)
        yield tok[:, :-1].contiguous(), tok[:, 1:].contiguous()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="tiny", choices=["tiny", "8b"])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--seq", type=int, default=None)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--max-grad-norm", type=float, default=1.0)
    ap.add_argument("--data", default=None)
    ap.add_argument("--save", default=None)
    ap.add_argument("--resume", default=None)
    ap.add_argument("--log-every", type=int, default=5)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0))) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": device} if cuda else {}))
    cfg = LlamaConfig.llama3_8b() if args.preset == "8b" else LlamaConfig.tiny()
    args.seq = args.seq or min(cfg.max_seq_len, 4096)
    model = Llama(cfg, device=device, dtype=torch.bfloat16 if cuda else torch.float32)
    model.reset_parameters(seed=0)
    engine = FSDPEngine(model, AdamWConfig(lr=args.lr), max_grad_norm=args.max_grad_norm)
    if args.resume:
        engine.load_checkpoint(args.resume)
    it = batches(args, cfg, rank, world, device)
    t0, seen = time.time(), 0
    for step in range(engine.step_count, engine.step_count + args.steps):
        tokens, targets = next(it)
        loss = engine.step(tokens, targets)
        seen += tokens.numel() * world
        if (step + 1) % args.log_every == 0:
            val = loss.float().clone()
            if world > 1:
                dist.all_reduce(val)
            if rank == 0:
                dt = time.time() - t0
                print(f"step {step + 1}: loss {val.item() / world:.4f}  grad-norm {float(engine.grad_norm):.3f}  "
                      f"{seen / dt:,.0f} tokens/s", flush=True)
    if args.save:
        engine.save_checkpoint(args.save)
        if rank == 0:
            print(f"saved sharded checkpoint to {args.save}", flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
