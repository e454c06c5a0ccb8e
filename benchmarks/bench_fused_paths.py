"""Device-timed microbenchmarks of the fused compute+collective paths against their rooflines.

Run with one rank per GPU:
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 benchmarks/bench_fused_paths.py

For every path it prints one JSON line with the fused time, the time of the unfused baseline
(NCCL collective + the same local kernel), and the achieved fraction of the roofline, defined as
the slower of FLOPs / measured GEMM peak and bytes over NVLink / measured peer-copy bandwidth
(770 GB/s per direction per GPU). Times are CUDA events, max over ranks.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.parallel.engine import AdamWConfig, FSDPEngine  # noqa: E402
from tensorplay_b200.parallel.tp import TPContext  # noqa: E402

NVLINK_GBS = 770.0


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 1590.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def report(rank, name, fused_ms, base_ms, flops, link_bytes, hbm_bytes, tf_peak, hbm_peak, which, extra=None):
    t_compute = flops / (tf_peak * 1e12) * 1e3
    t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    t_hbm = hbm_bytes / (hbm_peak * 1e9) * 1e3
    roof = max(t_compute, t_link, t_hbm)
    if rank == 0:
        out = {"path": name, "fused_ms": round(fused_ms, 4), "unfused_nccl_ms": round(base_ms, 4),
               "speedup_vs_unfused": round(base_ms / fused_ms, 3), "roofline_ms": round(roof, 4),
               "fraction_of_roofline": round(roof / fused_ms, 3),
               "bound": "compute" if roof == t_compute else ("nvlink" if roof == t_link else "hbm"),
               "peaks": which}
        if extra:
            out.update(extra)
        print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=8192)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    tf_peak, hbm_peak, which = peaks()
    torch.manual_seed(rank)

    # the engine creates the process-wide symmetric arena with head-room for the TP plans
    cfg = LlamaConfig(vocab_size=1024, hidden_size=4096, num_layers=2, num_heads=32, num_kv_heads=8,
                      head_dim=128, ffn_size=14336, max_seq_len=4096)
    model = Llama(cfg, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(0)
    eng = FSDPEngine(model, AdamWConfig(lr=1e-4), comm="symm" if world > 1 else "auto",
                     activation_checkpointing=True, symm_extra_bytes=3 << 30)
    # ---- tensor-parallel: all-gather -> GEMM (column-parallel) and GEMM -> reduce-scatter (row-parallel)
    tp = TPContext(arena_bytes=3 << 30)  # shares the engine's arena (one per process)
    M, H, F = args.tokens, 8192, 28672  # Llama-70B MLP: [tokens, 8192] x [2 * 28672 / tp, 8192]
    n_col = 2 * F // world
    x_loc = torch.randn(M // world, H, device=dev, dtype=torch.bfloat16)
    w_col = torch.randn(n_col, H, device=dev, dtype=torch.bfloat16) * 0.02
    xf = torch.empty(M, H, device=dev, dtype=torch.bfloat16)

    def ag_fused():
        with torch.no_grad():
            tp.all_gather_linear(x_loc, w_col)

    def ag_base():
        dist.all_gather_into_tensor(xf, x_loc)
        O.gemm(xf, w_col)

    t_f, t_b = timed(ag_fused, args.iters), timed(ag_base, args.iters)
    t_g = timed(lambda: O.gemm(xf, w_col), args.iters)
    report(rank, f"ag_gemm tp{world} [{M}x{H}]x[{n_col}x{H}]", t_f, t_b, 2.0 * M * H * n_col,
           (world - 1) * (M // world) * H * 2, 0, tf_peak, hbm_peak, which, {"local_gemm_only_ms": round(t_g, 4)})

    k_loc = F // world
    x_row = torch.randn(M, k_loc, device=dev, dtype=torch.bfloat16)
    w_row = torch.randn(H, k_loc, device=dev, dtype=torch.bfloat16) * 0.02
    y_loc = torch.empty(M // world, H, device=dev, dtype=torch.bfloat16)

    def rs_fused():
        with torch.no_grad():
            tp.linear_reduce_scatter(x_row, w_row)

    def rs_base():
        y = O.gemm(x_row, w_row)
        dist.reduce_scatter_tensor(y_loc, y)

    t_f, t_b = timed(rs_fused, args.iters), timed(rs_base, args.iters)
    t_g = timed(lambda: O.gemm(x_row, w_row), args.iters)
    report(rank, f"gemm_rs tp{world} [{M}x{k_loc}]x[{H}x{k_loc}]", t_f, t_b, 2.0 * M * k_loc * H,
           (world - 1) * (M // world) * H * 2, 0, tf_peak, hbm_peak, which, {"local_gemm_only_ms": round(t_g, 4)})

    # ---- FSDP parameter all-gather fused into the GEMM that consumes the weight: the Llama-8B gate/up projection,
    # [tokens, 4096] x gather([28672, 4096])^T, against (a) NCCL all-gather then GEMM and (b) the GEMM alone on an
    # already gathered weight (what an all-gather hidden a unit ahead leaves on the critical path)
    if world > 1:
        from tensorplay_b200.parallel.tp import WeightAGGemmPlan
        from tensorplay_b200.parallel.symm import SymmArena
        Mt, Kw, Nw = 4096, 4096, 28672
        plan = WeightAGGemmPlan(SymmArena._instance, Nw, Kw, rows_per_flag=256)
        plan.shard_view().normal_(0, 0.02)
        xw = torch.randn(Mt, Kw, device=dev, dtype=torch.bfloat16)
        w_full = torch.empty(Nw, Kw, device=dev, dtype=torch.bfloat16)
        w_shard = plan.shard_view().clone()
        out_w = torch.empty(Mt, Nw, device=dev, dtype=torch.bfloat16)

        def wag_fused():
            plan.run(xw, out=out_w)

        def wag_base():
            dist.all_gather_into_tensor(w_full, w_shard)
            O.gemm(xw, w_full, out=out_w)

        t_f, t_b = timed(wag_fused, args.iters), timed(wag_base, args.iters)
        t_g = timed(lambda: O.gemm(xw, w_full, out=out_w), args.iters)
        t_single = timed(lambda: O.gemm(xw, w_full, out=out_w, impl="single"), args.iters)
        ref = O.gemm(xw, w_full)
        plan.run(xw, out=out_w)
        torch.cuda.synchronize()
        err = ((out_w.float() - ref.float()).norm() / ref.float().norm()).item()
        report(rank, f"fsdp weight all-gather -> gemm fsdp{world} [{Mt}x{Kw}]x gather[{Nw}x{Kw}]", t_f, t_b,
               2.0 * Mt * Kw * Nw, (world - 1) * (Nw // world) * Kw * 2, 0, tf_peak, hbm_peak, which,
               {"local_gemm_only_ms": round(t_g, 4), "local_gemm_one_cta_kernel_ms": round(t_single, 4),
                "rel_err_vs_unfused": round(err, 6)})

    # ---- FSDP: parameter all-gather by peer pulls; reduce-scatter fused with scale + AdamW + bf16 emit
    u = max(eng.units, key=lambda t: t.padded)  # one transformer layer (218 M parameters)
    if world > 1:
        buf = eng.full_pool[0][: u.padded]
        nccl_buf = torch.empty(u.padded, device=dev, dtype=torch.bfloat16)
        shard_copy = u.shard.clone()

        g = eng.grad_pool[0][: u.padded]
        g.normal_()
        u._grad_slot = 0
        eng.step_count = 1
        gs = torch.empty(u.shard_numel, device=dev, dtype=torch.bfloat16)

        def gather_base():
            dist.all_gather_into_tensor(nccl_buf, shard_copy)

        def rs_adamw_base():
            dist.reduce_scatter_tensor(gs, g, op=dist.ReduceOp.AVG)
            O.adamw_flat_(u.master, u.exp_avg, u.exp_avg_sq, gs, shard_copy, **eng._adam_kwargs())

        t_gb, t_rb = timed(gather_base, args.iters), timed(rs_adamw_base, args.iters)
        comm = eng.comm
        raw = comm.arena.raw
        # every transport of the engine: copy engines; kernels with peer loads; the same kernels with the
        # in-switch reducing load; multicast push for the gather
        variants = [("ce", 1, "copy engines"), ("sm", 0, "peer loads")]
        if comm.arena.multicast:
            variants += [("sm", 1, "peer-load gather, multimem reduce"), ("mc", 1, "multicast-store gather, multimem reduce")]
        for transport, mc, label in variants:
            comm.transport = transport
            raw.tpb_symm_set_multicast(mc)
            if transport == "ce" and comm.staging is None:
                comm.staging = torch.empty(world * u.shard_numel, dtype=torch.bfloat16, device=dev)

            def gather_fused():
                comm.all_gather(u, buf)

            def rs_adamw_fused():
                comm.reduce_scatter_adamw(u, g, eng._adam_kwargs())
                comm.before_grad_reuse(0)

            t_f = timed(gather_fused, args.iters)
            report(rank, f"fsdp_all_gather {u.padded * 2 / 1e6:.0f} MB / {world} ranks", t_f, t_gb, 0.0,
                   (world - 1) * u.shard_numel * 2, u.padded * 2, tf_peak, hbm_peak, which, {"transport": label})
            t_f = timed(rs_adamw_fused, args.iters)
            # per rank: (world-1) slices of its shard leave every peer; AdamW streams 28 B per owned parameter
            report(rank, f"fsdp_rs_adamw {u.padded * 2 / 1e6:.0f} MB / {world} ranks", t_f, t_rb, 0.0,
                   (world - 1) * u.shard_numel * 2, u.shard_numel * (2 + 28), tf_peak, hbm_peak, which,
                   {"transport": label})
        raw.tpb_symm_set_multicast(1)
    torch.cuda.synchronize()
    O.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
