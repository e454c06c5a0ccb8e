"""Per-kernel device times of one expert-parallel MoE feed-forward (route, dispatch, grouped GEMMs,
SwiGLU, combine) and of its forward + backward, on one GPU.

The default shape is what one rank of the Qwen3-30B-A3B EP=8 configuration computes: 4096 tokens with
8 assignments each and 16 local experts of intermediate 768, i.e. 32768 expert rows of hidden 2048
(here every row stays on the local rank, so dispatch and combine move the same bytes through local
memory instead of NVLink).
Prints one JSON line; roofline fractions use the measured peaks (`--peak-tflops`, `--peak-gbs`).

    python benchmarks/bench_moe_layer.py
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_moe_layer.py

Under torchrun every rank brings `--tokens` tokens and owns `--experts` experts (N x experts in total), rows
cross NVLink, and the times are the maximum over the ranks (uniform random routing, so the load is balanced
and the numbers show the kernels, not the waiting for a slower rank).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.parallel.moe import MoEWorkspace, expert_parallel_ffn, grouped_gemm  # noqa: E402


def timed(fn, iters=10, warmup=3):
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    if dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096, help="tokens of this GPU")
    ap.add_argument("--experts", type=int, default=16)
    ap.add_argument("--top-k", type=int, default=8, help="assignments per token (tokens x k = expert rows)")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--inter", type=int, default=768)
    ap.add_argument("--peak-tflops", type=float, default=1620.4)
    ap.add_argument("--peak-gbs", type=float, default=6541.1)
    a = ap.parse_args()
    import torch.distributed as dist
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from tensorplay_b200.parallel.symm import SymmArena
        SymmArena(4 << 30)
    T, E, k, H, I = a.tokens, a.experts, a.top_k, a.hidden, a.inter
    torch.manual_seed(rank)
    x = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    idx = torch.randint(0, E * world, (T, k), device=dev)
    w = torch.rand(T, k, device=dev).to(torch.bfloat16)
    wgu = (0.02 * torch.randn(E, 2 * I, H, device=dev)).to(torch.bfloat16).requires_grad_()
    wd = (0.02 * torch.randn(E, H, I, device=dev)).to(torch.bfloat16).requires_grad_()
    ws = MoEWorkspace(T, k, H, E * world, capacity_factor=1.0 if world == 1 else 1.25)
    rows = T * k
    res = {"ranks": world, "tokens": T, "experts_per_rank": E, "top_k": k, "hidden": H, "inter": I,
           "expert_rows_per_rank": rows}

    dst_rank, dst_row, offs = ws.route(idx)
    res["route_ms"] = round(timed(lambda: ws.route(idx)), 4)
    res["dispatch_ms"] = round(timed(lambda: ws.dispatch(x, dst_rank, dst_row, ws.xbuf)), 4)
    gu = grouped_gemm(ws.xbuf, wgu, offs, workspace=ws.gws)
    res["gemm_gate_up_ms"] = round(timed(lambda: grouped_gemm(ws.xbuf, wgu, offs, workspace=ws.gws, out=gu)), 4)
    act = O.swiglu_packed(gu)
    res["swiglu_ms"] = round(timed(lambda: O.swiglu_packed(gu)), 4)
    res["gemm_down_ms"] = round(timed(lambda: grouped_gemm(act, wd, offs, out=ws.ybuf, workspace=ws.gws)), 4)
    wf = w.reshape(-1).float().contiguous()
    res["combine_ms"] = round(timed(lambda: ws.combine(ws.ybuf, dst_rank, dst_row, w=wf, tokens=T)), 4)
    dgu = torch.randn_like(gu)
    res["gemm_dgrad_ms"] = round(timed(lambda: grouped_gemm(dgu, wgu, offs, b_mn=True, out=ws.ybuf, workspace=ws.gws)), 4)
    wg = torch.empty(E, 2 * I, H, device=dev, dtype=torch.bfloat16)
    res["gemm_wgrad_ms"] = round(timed(lambda: grouped_gemm(dgu, ws.xbuf, offs, mode=1, out=wg, workspace=ws.gws)), 4)
    # rooflines
    fl_gu, fl_d = 2.0 * rows * H * 2 * I, 2.0 * rows * I * H
    res["gemm_gate_up_tflops"] = round(fl_gu / res["gemm_gate_up_ms"] / 1e9, 1)
    res["gemm_down_tflops"] = round(fl_d / res["gemm_down_ms"] / 1e9, 1)
    res["gemm_dgrad_tflops"] = round(fl_gu / res["gemm_dgrad_ms"] / 1e9, 1)
    res["gemm_wgrad_tflops"] = round(fl_gu / res["gemm_wgrad_ms"] / 1e9, 1)
    res["gemm_gate_up_of_peak"] = round(res["gemm_gate_up_tflops"] / a.peak_tflops, 3)
    res["gemm_down_of_peak"] = round(res["gemm_down_tflops"] / a.peak_tflops, 3)
    moved = 2.0 * rows * H * 2  # read + write of every routed row
    res["dispatch_gbs"] = round(moved / res["dispatch_ms"] / 1e6, 1)
    res["combine_gbs"] = round((rows * H * 2 + T * H * 2) / res["combine_ms"] / 1e6, 1)
    res["dispatch_of_hbm"] = round(res["dispatch_gbs"] / a.peak_gbs, 3)
    res["combine_of_hbm"] = round(res["combine_gbs"] / a.peak_gbs, 3)
    # whole op
    xg = x.clone().requires_grad_()
    wb = w.clone().requires_grad_()

    def fwd():
        with torch.no_grad():
            return expert_parallel_ffn(xg, idx, wb, wgu, wd, ws)

    def fwd_bwd():
        y = expert_parallel_ffn(xg, idx, wb, wgu, wd, ws)
        y.backward(torch.ones_like(y))
        xg.grad = wb.grad = wgu.grad = wd.grad = None

    res["ffn_forward_ms"] = round(timed(fwd), 4)
    res["ffn_forward_backward_ms"] = round(timed(fwd_bwd, iters=5), 4)
    res["ffn_fwd_bwd_model_tflops"] = round(3.0 * (fl_gu + fl_d) / res["ffn_forward_backward_ms"] / 1e9, 1)
    O.check_status()
    if world > 1:
        remote = (world - 1) / world * rows * H * 2   # bytes that cross NVLink per rank and direction
        res["dispatch_nvlink_gbs"] = round(remote / res["dispatch_ms"] / 1e6, 1)
        res["combine_nvlink_gbs"] = round(remote / res["combine_ms"] / 1e6, 1)
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
