"""Llama-3-8B-shape training on the composed layout TP x PP x FSDP (default 2 x 2 x world/4):
tensor-parallel blocks on the fused all-gather->GEMM / GEMM->reduce-scatter kernels, pipeline stages
under the 1F1B schedule with NCCL point-to-point (8 micro-batches of 1 x 4096 per data-parallel rank),
stage parameters sharded over the data-parallel group by ``fully_shard``, fused AdamW with fp32
master and state. Synthetic tokens, random-init weights; CUDA-event timing, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29515 benchmarks/bench_llama_3d.py --steps 3 --warmup 3

rank = pp * (dp * tp) + dp_rank * tp + tp_rank: tensor-parallel peers are neighbours.
``--cpu`` runs a tiny model on gloo ranks (a functional check of the same script).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tensorplay_b200 import ops  # noqa: E402
from tensorplay_b200.distributed.fsdp import fully_shard  # noqa: E402
from tensorplay_b200.distributed.pipelining import PipelineStage, Schedule1F1B  # noqa: E402
from tensorplay_b200.models.llama import LlamaConfig  # noqa: E402
from tensorplay_b200.models.llama_tp import LlamaTPStage, sync_replicated_grads  # noqa: E402
from tensorplay_b200.optim import AdamW  # noqa: E402
from tensorplay_b200.parallel.tp import TPContext  # noqa: E402


def make_groups(rank, tp, dp, pp):
    """Every rank creates every group in the same order; returns this rank's (tp, dp, pp) groups."""
    me = (rank // (dp * tp), (rank // tp) % dp, rank % tp)
    r = lambda p, d, t: p * dp * tp + d * tp + t  # noqa: E731
    mine = [None, None, None]
    for p in range(pp):
        for d in range(dp):
            g = dist.new_group([r(p, d, t) for t in range(tp)])
            if (p, d) == (me[0], me[1]):
                mine[0] = g
    for p in range(pp):
        for t in range(tp):
            g = dist.new_group([r(p, d, t) for d in range(dp)])
            if (p, t) == (me[0], me[2]):
                mine[1] = g
    for d in range(dp):
        for t in range(tp):
            g = dist.new_group([r(p, d, t) for p in range(pp)])
            if (d, t) == (me[1], me[2]):
                mine[2] = g
    return me, mine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if a.cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=96,
                               vocab_size=128, num_layers=a.layers, max_seq_len=a.seq)
        dtype = torch.float32
    else:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
        cfg = LlamaConfig.llama3_8b(max_seq_len=a.seq)
        cfg.num_layers = a.layers
        dtype = torch.bfloat16
    assert world % (a.tp * a.pp) == 0, "world must be a multiple of tp * pp"
    dp = world // (a.tp * a.pp)
    (pp_i, dp_i, tp_i), (tp_g, dp_g, pp_g) = make_groups(rank, a.tp, dp, a.pp)

    ctx = TPContext(group=tp_g, arena_bytes=2 << 30)
    stage_mod = LlamaTPStage(cfg, ctx, pp_i, a.pp, 1, a.seq, device=dev, dtype=dtype)
    stage_mod.reset_parameters(0)
    replicated = stage_mod.replicated_parameters()
    for blk in stage_mod.layers:
        fully_shard(blk, process_group=dp_g, reshard_after_forward=False)
    fully_shard(stage_mod, process_group=dp_g, reshard_after_forward=False)
    opt = AdamW(stage_mod.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)

    rows = a.seq // a.tp
    act = torch.empty(rows, cfg.hidden_size, dtype=dtype, device=dev)
    stage = PipelineStage(stage_mod, pp_i, a.pp, device=dev, group=pp_g,
                          input_args=None if pp_i == 0 else act, output_args=None if pp_i == a.pp - 1 else act)

    def loss_fn(logits, target):
        # mean over this rank's rows; the tensor-parallel ranks' parts add up to the sequence mean
        return ops.cross_entropy(logits.float() if a.cpu else logits, stage_mod.local_rows(target)) / a.tp

    sched = Schedule1F1B(stage, a.microbatches, loss_fn=loss_fn)
    g = torch.Generator().manual_seed(100 + dp_i)
    tokens = torch.randint(0, cfg.vocab_size, (a.microbatches, a.seq), generator=g).to(dev)
    targets = torch.randint(0, cfg.vocab_size, (a.microbatches, a.seq), generator=g).to(dev)
    last_loss = torch.zeros((), device=dev)
    # the step draws its tokens from the device generator: tensor-parallel peers (same stage, same
    # data-parallel rank) must draw the same ones
    torch.manual_seed(1000 + dp_i)

    def step():
        # fresh uniform tokens every step (a fixed batch is memorised within a few AdamW steps at
        # this width, and the loss would say nothing about the step being right)
        tokens.random_(0, cfg.vocab_size)
        targets.random_(0, cfg.vocab_size)
        opt.zero_grad(set_to_none=True)
        losses = []
        if a.pp == 1:
            sched.step(tokens, target=targets, losses=losses, return_outputs=False)
            last_loss.copy_(torch.stack(losses).sum() / a.microbatches)
        elif pp_i == 0:
            sched.step(tokens)
        elif pp_i == a.pp - 1:
            sched.step(target=targets, losses=losses, return_outputs=False)
            last_loss.copy_(torch.stack(losses).sum() / a.microbatches)
        else:
            sched.step()
        sync_replicated_grads(stage_mod, replicated, tp_g)
        opt.step()

    for _ in range(a.warmup):
        step()
    dist.barrier()
    if not a.cpu:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
        ops.check_status()
    else:
        import time
        t0 = time.perf_counter()
        for _ in range(a.steps):
            step()
        ms = torch.tensor([(time.perf_counter() - t0) * 1e3 / a.steps])
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    loss = last_loss.clone()
    dist.all_reduce(loss)            # only the last stage contributed: sum over its tp x dp ranks
    loss = loss.item() / dp
    tokens_per_step = dp * a.microbatches * a.seq
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/s/box, Llama-3-8B-shape TP x PP x FSDP bf16, max over ranks",
            "value": round(tokens_per_step / (ms.item() * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
            "ms_per_step": round(ms.item(), 3), "steps": a.steps, "warmup": a.warmup, "loss": round(loss, 4),
            "dtype": "fp32 (cpu check)" if a.cpu else "bf16", "data": "synthetic",
            "config": {"model": "tiny" if a.cpu else "Llama-3-8B-shape", "layers": a.layers,
                       "parallelism": f"tp{a.tp} x pp{a.pp} (1F1B, {a.microbatches} micro-batches) x fsdp{dp}",
                       "global_batch": dp * a.microbatches, "seq_len": a.seq,
                       "optimizer": "AdamW fp32 state + fp32 master"}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
