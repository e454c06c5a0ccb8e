"""Data-parallel training when the ranks have different numbers of batches: ``DistributedDataParallel`` with the ZeRO-1
optimizer inside a ``Join`` context. A rank that runs out of data keeps answering the other ranks' collectives (its
gradient contribution is zero, its optimizer shard still steps), and at the end every rank holds the same parameters.

    python -m tensorplay_b200.distributed.run --nproc-per-node 2 examples/train_ddp_uneven.py [--device cpu]

Runs on CPU ranks (gloo) as well as on GPUs (NCCL).
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200.distributed.algorithms import Join  # noqa: E402
from tensorplay_b200.distributed.ddp import DistributedDataParallel as DDP  # noqa: E402
from tensorplay_b200.distributed.optim import ZeroRedundancyOptimizer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--batches", type=int, default=6, help="batches on rank 0; rank r has r more")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if a.device == "cuda":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl" if a.device == "cuda" else "gloo")
    dev = torch.device(a.device, torch.cuda.current_device()) if a.device == "cuda" else torch.device("cpu")

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 1)).to(dev)
    ddp = DDP(model, bucket_cap_mb=0.01, comm="torch")
    opt = ZeroRedundancyOptimizer(model.parameters(), torch.optim.AdamW, lr=3e-3)
    owned = sum(p.numel() for g in opt.optim.param_groups for p in g["params"])
    gen = torch.Generator().manual_seed(100 + rank)
    w_true = torch.linspace(-1, 1, 32)

    n_batches = a.batches + rank
    with Join([ddp, opt]):
        for step in range(n_batches):
            x = torch.randn(64, 32, generator=gen)
            y = (x @ w_true).unsqueeze(1)
            loss = (ddp(x.to(dev)) - y.to(dev)).pow(2).mean()
            model.zero_grad(set_to_none=False)
            loss.backward()
            opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    same = bool(torch.equal(flat, ref))
    print(f"rank {rank}: {n_batches} batches, optimizer state for {owned} of {flat.numel()} parameters, "
          f"last loss {float(loss.detach()):.4f}, parameters equal to rank 0: {same}", flush=True)
    dist.destroy_process_group()
    if not same:
        sys.exit(1)


if __name__ == "__main__":
    main()
