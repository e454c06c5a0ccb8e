"""torchrun worker: fused all-gather->GEMM and GEMM->reduce-scatter vs NCCL + fp32 matmul."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.parallel.tp import TPContext  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    tp = TPContext(arena_bytes=1 << 30)
    for p in list(tp._ag.values()) + list(tp._rs.values()):
        p.wait_s = 10.0
    res = {"rank": rank, "ok": True, "msgs": []}
    torch.manual_seed(100 + rank)
    M, K, N = 1024 * world, 1024, 768
    for it in range(3):  # repeated calls exercise buffer rotation and epochs
        x_local = torch.randn(M // world, K, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16, requires_grad=True) * 0.05
        w = w.detach().requires_grad_()
        y = tp.all_gather_linear(x_local, w)
        gy = torch.randn_like(y)
        y.backward(gy)
        # reference
        xf = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(xf, x_local.detach())
        yr = xf.float() @ w.detach().float().t()
        dxr_full = gy.float() @ w.detach().float()
        dist.all_reduce(dxr_full)
        dxr = dxr_full[rank * (M // world): (rank + 1) * (M // world)]
        dwr = gy.float().t() @ xf.float()
        for name, a, b, tol in (("ag_y", y, yr, 1e-2), ("ag_dx", x_local.grad, dxr, 1.5e-2), ("ag_dw", w.grad, dwr, 1e-2)):
            e = rel(a, b)
            if not e < tol:
                res["ok"] = False
                res["msgs"].append(f"it{it} {name} rel {e}")
        # row-parallel: x [M, K_local] @ w [N, K_local]^T summed over ranks, rows scattered
        x2 = torch.randn(M, K, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w2 = (torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.05).requires_grad_()
        y2 = tp.linear_reduce_scatter(x2, w2)
        gy2 = torch.randn_like(y2)
        y2.backward(gy2)
        full = x2.detach().float() @ w2.detach().float().t()
        dist.all_reduce(full)
        y2r = full[rank * (M // world): (rank + 1) * (M // world)]
        gfull = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(gfull, gy2)
        dx2r = gfull.float() @ w2.detach().float()
        dw2r = gfull.float().t() @ x2.detach().float()
        for name, a, b, tol in (("rs_y", y2, y2r, 1.5e-2), ("rs_dx", x2.grad, dx2r, 1e-2), ("rs_dw", w2.grad, dw2r, 1e-2)):
            e = rel(a, b)
            if not e < tol:
                res["ok"] = False
                res["msgs"].append(f"it{it} {name} rel {e}")
    torch.cuda.synchronize()
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
