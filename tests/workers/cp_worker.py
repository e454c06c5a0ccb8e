"""torchrun worker: ring attention (context parallel) on GPUs vs full-sequence fp32 attention,
and the clipped (two-phase) engine step over symmetric memory vs the NCCL path."""
import copy
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.ops.attention import attention_reference  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402
from tensorplay_b200.parallel.cp import context_parallel_shard, ring_attention  # noqa: E402
from tensorplay_b200.parallel.symm import SymmArena  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    res = {"rank": rank, "ok": True, "msgs": []}

    # ---- clipped engine step: symmetric-memory reduce-only kernel vs NCCL reduce-scatter
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn_size=512,
                           vocab_size=512, num_layers=2)
    base = Llama(cfg, device=dev, dtype=torch.bfloat16)
    base.reset_parameters(0)
    g = torch.Generator().manual_seed(5)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 128), generator=g).to(dev)
    tgts = torch.randint(0, cfg.vocab_size, (world, 2, 128), generator=g).to(dev)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    states, norms = {}, {}
    for kind in ("symm", "torch"):
        eng = FSDPEngine(copy.deepcopy(base), ocfg, comm=kind, max_grad_norm=0.05, symm_extra_bytes=1 << 30)
        ns = []
        for _ in range(3):
            eng.step(toks[rank], tgts[rank])
            ns.append(float(eng.grad_norm))
        states[kind], norms[kind] = eng.gather_full_state(), ns
    for a, b in zip(norms["symm"], norms["torch"]):
        if not abs(a - b) < 2e-2 * max(b, 1e-3):
            res["ok"] = False
            res["msgs"].append(f"grad norm symm {a} vs nccl {b}")
    if not norms["symm"][0] > 0.05:
        res["ok"] = False
        res["msgs"].append("clip was not active")
    for n in states["torch"]:
        e = rel(states["symm"][n], states["torch"][n])
        if not e < 5e-3:
            res["ok"] = False
            res["msgs"].append(f"clipped params {n} rel {e}")

    # ---- ring attention
    assert SymmArena._instance is not None
    for causal in (True, False):
        torch.manual_seed(1)
        B, T, Hq, Hkv, D = 2, 256 * world, 8, 2, 128
        q = torch.randn(B, T, Hq, D, device=dev, dtype=torch.bfloat16)
        k = torch.randn(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
        v = torch.randn(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
        go = torch.randn(B, T, Hq, D, device=dev, dtype=torch.bfloat16)
        qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
        ref = attention_reference(qr, kr, vr, causal)
        ref.backward(go.float())
        ql, kl, vl, gl = (t.detach().requires_grad_() for t in context_parallel_shard([q, k, v, go], [1, 1, 1, 1]))
        for it in range(2):  # twice: arena buffers and epochs are reused
            for t in (ql, kl, vl):
                t.grad = None
            out = ring_attention(ql, kl, vl, causal)
            out.backward(gl.detach())
        lo, hi = rank * (T // world), (rank + 1) * (T // world)
        for name, a, b in (("o", out, ref[:, lo:hi]), ("dq", ql.grad, qr.grad[:, lo:hi]),
                           ("dk", kl.grad, kr.grad[:, lo:hi]), ("dv", vl.grad, vr.grad[:, lo:hi])):
            e = rel(a, b)
            if not e < 2e-2:
                res["ok"] = False
                res["msgs"].append(f"ring causal={causal} {name} rel {e}")
    # ---- load-balanced (head-tail) sharding for the causal mask
    torch.manual_seed(2)
    B, T, Hq, Hkv, D = 1, 256 * 2 * world, 8, 2, 128
    q = torch.randn(B, T, Hq, D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
    go = torch.randn(B, T, Hq, D, device=dev, dtype=torch.bfloat16)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, True)
    ref.backward(go.float())
    ql, kl, vl, gl = (t.detach().requires_grad_() for t in
                      context_parallel_shard([q, k, v, go], [1, 1, 1, 1], load_balance=True))
    out = ring_attention(ql, kl, vl, True, load_balance=True)
    out.backward(gl.detach())
    wants = context_parallel_shard([ref.detach(), qr.grad, kr.grad, vr.grad], [1, 1, 1, 1], load_balance=True)
    for name, a, b in zip(("o", "dq", "dk", "dv"), (out, ql.grad, kl.grad, vl.grad), wants):
        e = rel(a, b)
        if not e < 2e-2:
            res["ok"] = False
            res["msgs"].append(f"ring zigzag {name} rel {e}")
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
