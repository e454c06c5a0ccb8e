"""torchrun worker: sharded engine on peer-memory kernels vs the NCCL path vs a dense fp32 run."""
import copy
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, head_dim=64, ffn_size=512,
                           vocab_size=512, num_layers=3)
    base = Llama(cfg, device=dev, dtype=torch.bfloat16)
    base.reset_parameters(seed=7)
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    g = torch.Generator().manual_seed(11)
    toks = torch.randint(0, cfg.vocab_size, (world, 2, 128), generator=g)
    tgts = torch.randint(0, cfg.vocab_size, (world, 2, 128), generator=g)
    steps = 4
    out = {}
    for kind in ("torch", "symm"):
        m = copy.deepcopy(base)
        eng = FSDPEngine(m, ocfg, comm=kind, activation_checkpointing=True)
        if kind == "symm":
            eng.comm.wait_s = 10.0
        losses = []
        for _ in range(steps):
            losses.append(float(eng.step(toks[rank].to(dev), tgts[rank].to(dev))))
        torch.cuda.synchronize()
        O.check_status()
        state = eng.gather_full_state()
        out[kind] = (losses, state)
    # dense fp32 reference on the concatenated batch
    ref = copy.deepcopy(base).float()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = ref(toks.flatten(0, 1).to(dev), tgts.flatten(0, 1).to(dev))
        loss.backward()
        opt.step()
        ref_losses.append(float(loss))
    res = {"rank": rank, "ok": True, "msgs": []}
    for kind in ("torch", "symm"):
        losses, state = out[kind]
        mean_loss = torch.tensor(losses, device=dev)
        dist.all_reduce(mean_loss)
        mean_loss /= world
        for a, b in zip(mean_loss.tolist(), ref_losses):
            if abs(a - b) > 0.06:
                res["ok"] = False
                res["msgs"].append(f"{kind}: loss {a} vs ref {b}")
        worst = 0.0
        for n, p in ref.named_parameters():
            d = (state[n] - p.detach()).abs().max().item()
            worst = max(worst, d)
        res[kind + "_max_param_diff"] = worst
        if worst > 8e-3:
            res["ok"] = False
            res["msgs"].append(f"{kind}: param diff {worst}")
    # the two sharded paths must agree closely with each other
    d = max((out["torch"][1][n] - out["symm"][1][n]).abs().max().item() for n in out["symm"][1])
    res["symm_vs_torch"] = d
    if d > 4e-3:
        res["ok"] = False
        res["msgs"].append(f"symm vs torch {d}")
    print("RESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
