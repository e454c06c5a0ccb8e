"""Llama-3-70B-shape tensor-parallel inference (TP = world size), bf16 weights and KV cache:
prefill of batch 8 x 4096 prompt tokens (tokens/s) and greedy decode of batch 64 x N new tokens
(per-token latency p50 from CUDA events). Synthetic prompts, random-init weights.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/bench_tp_inference.py [--layers 80] [--new-tokens 512]
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.llama import LlamaConfig  # noqa: E402
from tensorplay_b200.models.llama_tp import LlamaTP  # noqa: E402
from tensorplay_b200.ops.gemm import enable_splitk  # noqa: E402
from tensorplay_b200.parallel.tp import TPContext  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--new-tokens", type=int, default=512)
    ap.add_argument("--prefill-batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--decode-batch", type=int, default=64)
    ap.add_argument("--model", default="70b", choices=["70b", "8b", "tiny"])
    ap.add_argument("--decode-layout", default="replicated", choices=["replicated", "sequence"],
                    help="replicated activations + one-launch all-reduce/residual/norm, or rows sharded over the ranks "
                         "with fused all-gather / reduce-scatter GEMMs")
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = {"70b": LlamaConfig.llama3_70b, "8b": LlamaConfig.llama3_8b,
           "tiny": lambda **k: LlamaConfig.tiny(num_heads=8, num_kv_heads=8, head_dim=128, hidden_size=1024, ffn_size=2048, **k)}[a.model](
        max_seq_len=a.prompt + a.new_tokens)
    cfg.num_layers = a.layers
    tp = TPContext(arena_bytes=6 << 30)
    enable_splitk()
    model = LlamaTP(cfg, tp, device=dev, dtype=torch.bfloat16)
    model.reset_parameters(0)
    model.decode_layout = a.decode_layout
    g = torch.Generator().manual_seed(0)
    # ---- prefill: batch x prompt
    prompts = torch.randint(0, cfg.vocab_size, (a.prefill_batch, a.prompt), generator=g).to(dev)
    model.allocate_cache(max(a.prefill_batch, a.decode_batch), a.prompt + a.new_tokens)
    for _ in range(2):
        model.prefill(prompts)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    nxt = model.prefill(prompts)
    e1.record()
    torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1)
    # ---- decode: batch 64 continuing from a (synthetic) cache of `prompt` tokens
    last = torch.randint(0, cfg.vocab_size, (a.decode_batch,), generator=g).to(dev)
    for i in range(3):
        last = model.decode_step(last, a.prompt + i)
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(True) for _ in range(a.new_tokens + 1)]
    evs[0].record()
    for i in range(a.new_tokens):
        last = model.decode_step(last, a.prompt + i)
        evs[i + 1].record()
    torch.cuda.synchronize()
    O.check_status()
    lat = [evs[i].elapsed_time(evs[i + 1]) for i in range(a.new_tokens)]
    t = torch.tensor([prefill_ms, statistics.median(lat)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"config": f"Llama-3-{a.model}-shape TP={world} inference, {a.layers} layers, bf16",
                          "prefill_tokens_per_s": round(a.prefill_batch * a.prompt / (float(t[0]) / 1e3), 1),
                          "prefill_ms": round(float(t[0]), 2),
                          "decode_layout": a.decode_layout,
                          "decode_batch": a.decode_batch, "decode_ms_per_token_p50": round(float(t[1]), 3),
                          "decode_tokens_per_s": round(a.decode_batch / (float(t[1]) / 1e3), 1),
                          "new_tokens": a.new_tokens, "data": "synthetic", "timing": "CUDA events, max over ranks"}),
              flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
