"""torchrun worker: tensor-parallel Llama (prefill + cached decode) equals the dense model."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import tensorplay_b200.ops as O  # noqa: E402
from tensorplay_b200.models.llama import Llama, LlamaConfig  # noqa: E402
from tensorplay_b200.models.llama_tp import LlamaTP  # noqa: E402
from tensorplay_b200.ops.gemm import enable_splitk  # noqa: E402
from tensorplay_b200.parallel.tp import TPContext  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = LlamaConfig.tiny(hidden_size=512, num_heads=8, num_kv_heads=4, head_dim=64, ffn_size=1024,
                           vocab_size=1024, num_layers=2, max_seq_len=512)
    tp = TPContext(arena_bytes=1 << 30)
    enable_splitk()
    dense = Llama(cfg, device=dev, dtype=torch.bfloat16)
    dense.reset_parameters(seed=3)
    m = LlamaTP(cfg, tp, device=dev, dtype=torch.bfloat16)
    # shard the dense weights
    w, r = world, rank
    D, Hq, Hkv, F = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.ffn_size
    with torch.no_grad():
        m.embed.copy_(dense.embed)
        m.final_norm.copy_(dense.final_norm)
        vs = m.vshard
        m.lm_head.zero_()
        n = min(vs, cfg.vocab_size - r * vs)
        m.lm_head[:n].copy_(dense.lm_head[r * vs: r * vs + n])
        for lt, ld in zip(m.layers, dense.layers):
            lt.attn_norm.copy_(ld.attn_norm)
            lt.ffn_norm.copy_(ld.ffn_norm)
            q = ld.wqkv[: Hq * D].view(Hq, D, -1)[r * lt.hq: (r + 1) * lt.hq].reshape(lt.hq * D, -1)
            k = ld.wqkv[Hq * D: (Hq + Hkv) * D].view(Hkv, D, -1)[r * lt.hkv: (r + 1) * lt.hkv].reshape(lt.hkv * D, -1)
            v = ld.wqkv[(Hq + Hkv) * D:].view(Hkv, D, -1)[r * lt.hkv: (r + 1) * lt.hkv].reshape(lt.hkv * D, -1)
            lt.wqkv.copy_(torch.cat((q, k, v), 0))
            lt.wo.copy_(ld.wo[:, r * lt.hq * D: (r + 1) * lt.hq * D])
            g, u = ld.w_gate_up[:F], ld.w_gate_up[F:]
            lt.w_gate_up.copy_(torch.cat((g[r * lt.ff: (r + 1) * lt.ff], u[r * lt.ff: (r + 1) * lt.ff]), 0))
            lt.w_down.copy_(ld.w_down[:, r * lt.ff: (r + 1) * lt.ff])
    B, T = 4, 128
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(dev)
    res = {"rank": rank, "ok": True, "msgs": []}
    with torch.no_grad():
        ref_logits = dense(toks).float()               # [B, T, V]
        m.allocate_cache(B, T + 8)
        x = m.hidden(toks, 0, use_cache=True)
        h_last = m.last_token_hidden(x, B, T)
        nxt = m.greedy_next(h_last)
        ref_next = ref_logits[:, -1].argmax(-1)
        # compare hidden states through the logits of the local vocabulary shard
        hl = O.rms_norm(h_last, m.final_norm, cfg.rms_eps)
        lg = O.linear(hl, m.lm_head).float()[:, :n]
        e = ((lg - ref_logits[:, -1, r * vs: r * vs + n]).norm() / ref_logits[:, -1].norm()).item()
        if e > 3e-2:
            res["ok"] = False
            res["msgs"].append(f"prefill logits rel {e}")
        agree = (nxt == ref_next).float().mean().item()
        # decode 4 tokens with the cache vs dense recompute
        # both decode layouts: replicated activations with the one-launch all-reduce + residual + norm (the default),
        # and rows sharded over the ranks with the fused all-gather / reduce-scatter GEMMs
        for layout in ("replicated", "sequence"):
            m.decode_layout = layout
            m._graph = None
            seq = torch.cat((toks, ref_next[:, None]), 1)
            last = ref_next
            for i in range(4):   # the first step runs eagerly and is captured, the others replay the graph
                nx = m.decode_step(last, T + i)
                ref_nx = dense(seq).float()[:, -1].argmax(-1)
                a = (nx == ref_nx).float().mean().item()
                if a < 0.75:
                    res["msgs"].append(f"{layout} decode step {i}: agreement {a}")
                agree = min(agree, a)
                seq = torch.cat((seq, ref_nx[:, None]), 1)
                last = ref_nx
        res["agree"] = agree
        if agree < 0.75:
            res["ok"] = False
            res["msgs"].append(f"greedy agreement {agree}")
    torch.cuda.synchronize()
    try:
        O.check_status()
    except Exception as ex:
        res["ok"] = False
        res["msgs"].append(str(ex))
    print("RESULT " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
