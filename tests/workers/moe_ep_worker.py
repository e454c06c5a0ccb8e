"""torchrun worker: expert-parallel FFN over peer memory vs a dense all-gathered reference."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.parallel.moe import (MoEWorkspace, expert_ffn_reference, expert_parallel_ffn,  # noqa: E402
                                          topk_route)


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    T, H, I, E, k = 1024, 512, 256, 8 * world, 4
    El = E // world
    ws = MoEWorkspace(T, k, H, E, wait_s=10.0, capacity_factor=3.0)
    torch.manual_seed(50 + rank)
    res = {"rank": rank, "ok": True, "msgs": []}
    wgu = (torch.randn(El, 2 * I, H, device=dev, dtype=torch.bfloat16) * 0.05).requires_grad_()
    wd = (torch.randn(El, H, I, device=dev, dtype=torch.bfloat16) * 0.05).requires_grad_()
    for it in range(2):
        x = torch.randn(T, H, device=dev, dtype=torch.bfloat16, requires_grad=True)
        idx, w, _ = topk_route(torch.randn(T, E, device=dev), k)
        w = w.to(torch.bfloat16).requires_grad_()
        wgu.grad = wd.grad = None
        y = expert_parallel_ffn(x, idx, w, wgu, wd, ws)
        g = torch.randn_like(y)
        y.backward(g)
        torch.cuda.synchronize()
        xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        gur, dr = wgu.detach().float().requires_grad_(), wd.detach().float().requires_grad_()
        yr = expert_ffn_reference(xr, idx, wr, gur, dr)
        yr.backward(g.float())  # all_gather's backward sums the expert-weight grads over ranks
        for name, a, b, tol in (("y", y, yr, 1.5e-2), ("dx", x.grad, xr.grad, 2e-2), ("dw", w.grad, wr.grad, 2e-2),
                                ("dwgu", wgu.grad, gur.grad, 2e-2), ("dwd", wd.grad, dr.grad, 2e-2)):
            e = rel(a, b)
            if not e < tol:
                res["ok"] = False
                res["msgs"].append(f"it{it} {name} rel {e}")
    try:
        O.check_status()
    except Exception as e:
        res["ok"] = False
        res["msgs"].append(str(e))
    print("RESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
