"""Proxy baseline: the same Llama-3-8B-shape training step run through stock PyTorch - FSDP2
(``torch.distributed.fsdp.fully_shard``: copy-in -> ncclAllGather -> copy-out, ncclReduceScatter),
cuBLAS GEMMs, SDPA flash attention, activation checkpointing, fused torch AdamW - i.e. the
algorithm the reference executes (tensorplay/distributed/fsdp/_fully_shard/_fsdp_collectives.py:
337-690), used as the yard-stick because the reference itself cannot be built offline.
Prints one JSON line in bench.py's format with ``"impl": "proxy-torch-fsdp2"``.

    python baseline/proxy_torch_fsdp.py --steps 3 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... baseline/proxy_torch_fsdp.py --gpus N
"""
import argparse
import json
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


class Block(nn.Module):
    def __init__(self, H, Hq, Hkv, D, FF, eps):
        super().__init__()
        self.Hq, self.Hkv, self.D = Hq, Hkv, D
        self.n1 = nn.RMSNorm(H, eps=eps)
        self.n2 = nn.RMSNorm(H, eps=eps)
        self.qkv = nn.Linear(H, (Hq + 2 * Hkv) * D, bias=False)
        self.o = nn.Linear(Hq * D, H, bias=False)
        self.gu = nn.Linear(H, 2 * FF, bias=False)
        self.down = nn.Linear(FF, H, bias=False)

    def forward(self, x, cos, sin):
        B, T, H = x.shape
        qkv = self.qkv(self.n1(x)).view(B, T, self.Hq + 2 * self.Hkv, self.D)
        q, k, v = qkv[:, :, :self.Hq], qkv[:, :, self.Hq:self.Hq + self.Hkv], qkv[:, :, self.Hq + self.Hkv:]

        def rope(t):
            a, b = t[..., : self.D // 2].float(), t[..., self.D // 2:].float()
            return torch.cat((a * cos - b * sin, b * cos + a * sin), -1).to(t.dtype)
        q, k = rope(q), rope(k)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=True).transpose(1, 2).reshape(B, T, -1)
        x = x + self.o(o)
        g, u = self.gu(self.n2(x)).chunk(2, -1)
        return x + self.down(F.silu(g) * u)


def _selective_contexts():
    from torch.utils.checkpoint import CheckpointPolicy, create_selective_checkpoint_contexts
    keep = {torch.ops.aten.mm.default, torch.ops.aten.addmm.default, torch.ops.aten.bmm.default,
            torch.ops.aten._scaled_dot_product_flash_attention.default,
            torch.ops.aten._scaled_dot_product_cudnn_attention.default,
            torch.ops.aten._scaled_dot_product_efficient_attention.default}

    def policy(ctx, op, *args, **kwargs):
        return CheckpointPolicy.MUST_SAVE if op in keep else CheckpointPolicy.PREFER_RECOMPUTE

    return create_selective_checkpoint_contexts(policy)


class Model(nn.Module):
    def __init__(self, V=128256, H=4096, L=32, Hq=32, Hkv=8, D=128, FF=14336, eps=1e-5, theta=5e5, T=4096):
        super().__init__()
        self.emb = nn.Embedding(V, H)
        self.layers = nn.ModuleList([Block(H, Hq, Hkv, D, FF, eps) for _ in range(L)])
        self.norm = nn.RMSNorm(H, eps=eps)
        self.head = nn.Linear(H, V, bias=False)
        inv = 1.0 / (theta ** (torch.arange(0, D, 2).float() / D))
        ang = torch.outer(torch.arange(T).float(), inv)
        self.register_buffer("cos", ang.cos()[None, :, None, :], persistent=False)
        self.register_buffer("sin", ang.sin()[None, :, None, :], persistent=False)

    ac = "full"  # "selective": keep matmul and attention outputs, recompute the rest (torch's policy API)

    def forward(self, tok, tgt):
        x = self.emb(tok)
        for l in self.layers:
            if self.ac == "selective":
                x = checkpoint(l, x, self.cos, self.sin, use_reentrant=False, context_fn=_selective_contexts)
            else:
                x = checkpoint(l, x, self.cos, self.sin, use_reentrant=False)
        logits = self.head(self.norm(x))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), tgt.reshape(-1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--ac", default="full", choices=["full", "selective"])
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    with torch.device(dev):
        model = Model(L=a.layers).to(torch.bfloat16)
        model.ac = a.ac
    for p in model.parameters():
        if p.dim() > 1:
            nn.init.normal_(p, std=0.02)
    if world > 1:
        from torch.distributed.fsdp import fully_shard
        for l in model.layers:
            fully_shard(l)
        fully_shard(model)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    T = 4096
    tok = torch.randint(0, 128256, (1, T), device=dev)
    tgt = torch.randint(0, 128256, (1, T), device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        loss = model(tok, tgt)
        loss.backward()
        opt.step()
        return loss
    for _ in range(a.warmup):
        step()
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
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0])
    if rank == 0:
        print(json.dumps({"impl": "proxy-torch-fsdp2", "metric": "train tokens/s/box, Llama-3-8B-shape FSDP bf16",
                          "note": "bf16 parameters and bf16 AdamW state (torch fused AdamW on bf16 params); no fp32 master",
                          "value": round(world * T * a.steps / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world,
                          "ms_per_step": round(ms / a.steps, 3), "loss": round(float(loss), 4),
                          "layers": a.layers, "activation_checkpointing": a.ac}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
