"""Tensor-parallel building blocks and the tensor-parallel Llama on two gloo ranks (CPU oracle path)."""
import torch

from tests.distutil import run_ranks


def _tp_linear_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.parallel.tp import TPContext
    tp = TPContext()
    torch.manual_seed(0)
    M, K, N = 8 * world, 16, 12
    x_full = torch.randn(M, K)
    w_col = torch.randn(N * world, K)            # column-parallel: rows of W sharded
    rows = M // world
    x_local = x_full[rank * rows: (rank + 1) * rows].clone().requires_grad_()
    w_shard = w_col[rank * N: (rank + 1) * N].clone().requires_grad_()
    y = tp.all_gather_linear(x_local, w_shard)   # [M, N]
    torch.testing.assert_close(y, x_full @ w_shard.t(), rtol=1e-5, atol=1e-5)
    gy = torch.randn(M, N, generator=torch.Generator().manual_seed(7 + rank))
    y.backward(gy)
    # dx_local = rows of sum_r (gy_r @ W_r)
    parts = [torch.zeros(M, N) for _ in range(world)]
    dist.all_gather(parts, gy)
    dx_full = sum(parts[r] @ w_col[r * N: (r + 1) * N] for r in range(world))
    torch.testing.assert_close(x_local.grad, dx_full[rank * rows: (rank + 1) * rows], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(w_shard.grad, gy.t() @ x_full, rtol=1e-4, atol=1e-5)
    # row-parallel: K sharded, output rows scattered
    w_row = torch.randn(N, K * world)
    x2 = torch.randn(M, K * world)
    y2 = tp.linear_reduce_scatter(x2[:, rank * K: (rank + 1) * K].contiguous(), w_row[:, rank * K: (rank + 1) * K].contiguous())
    torch.testing.assert_close(y2, (x2 @ w_row.t())[rank * rows: (rank + 1) * rows], rtol=1e-4, atol=1e-4)
    dist.barrier()
    return True


def test_tp_linears_match_dense_math():
    assert all(run_ranks(_tp_linear_worker, 2))


def _tp_llama_worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200.models.llama import Llama, LlamaConfig
    from tensorplay_b200.models.llama_tp import LlamaTP
    from tensorplay_b200.parallel.tp import TPContext
    cfg = LlamaConfig.tiny(hidden_size=64, num_heads=4, num_kv_heads=2, head_dim=16, ffn_size=96, vocab_size=100,
                           num_layers=2, max_seq_len=64)
    tp = TPContext()
    dense = Llama(cfg)
    dense.reset_parameters(seed=3)
    m = LlamaTP(cfg, tp)
    r, D, Hq, Hkv, F = rank, cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.ffn_size
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
    B, T = 2, 10
    toks = torch.randint(0, cfg.vocab_size, (B, T), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref_logits = dense(toks)
        m.allocate_cache(B, T + 4)
        nxt = m.prefill(toks)
        assert torch.equal(nxt, ref_logits[:, -1].argmax(-1))
        seq = torch.cat((toks, nxt[:, None]), 1)
        last = nxt
        for i in range(3):  # cached decode equals dense recomputation
            last = m.decode_step(last, T + i)
            ref = dense(seq)[:, -1].argmax(-1)
            assert torch.equal(last, ref), (i, last, ref)
            seq = torch.cat((seq, ref[:, None]), 1)
    dist.barrier()
    return True


def test_tensor_parallel_llama_equals_dense_on_two_ranks():
    assert all(run_ranks(_tp_llama_worker, 2))
