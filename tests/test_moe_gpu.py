"""Grouped tcgen05 GEMM and the single-rank expert-parallel path against PyTorch references."""
import pytest
import torch

import tensorplay_b200.ops as O
from tensorplay_b200.parallel.moe import (MoEWorkspace, expert_ffn_reference, expert_parallel_ffn,
                                          grouped_gemm, topk_route)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _offs(counts):
    o = [0]
    for c in counts:
        o.append(o[-1] + (c + 127) // 128 * 128)
    return o


@pytest.mark.parametrize("counts,N,K", [([128, 0, 256, 384], 256, 128), ([100, 300, 7, 0, 129], 1536, 2048),
                                        ([512] * 4, 768, 2048)])
def test_grouped_gemm_modes(counts, N, K):
    torch.manual_seed(0)
    G = len(counts)
    o = _offs(counts)
    rows = o[-1]
    a = torch.zeros(rows, K, device=DEV, dtype=torch.bfloat16)
    for e, c in enumerate(counts):
        a[o[e]: o[e] + c] = torch.randn(c, K, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(G, N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    offs = torch.tensor(o, dtype=torch.int32, device=DEV)
    y = grouped_gemm(a, w, offs)
    O.check_status()
    for e, c in enumerate(counts):
        if c:
            ref = a[o[e]: o[e] + c].float() @ w[e].float().t()
            assert _rel(y[o[e]: o[e] + c], ref) < 6e-3, e
    # input gradient form: dx = dy @ W[e]
    dy = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16)
    for e, c in enumerate(counts):
        dy[o[e]: o[e] + c] = torch.randn(c, N, device=DEV, dtype=torch.bfloat16)
    dx = grouped_gemm(dy, w, offs, b_mn=True)
    for e, c in enumerate(counts):
        if c:
            assert _rel(dx[o[e]: o[e] + c], dy[o[e]: o[e] + c].float() @ w[e].float()) < 6e-3, e
    # weight gradient form: dW[e] = dy_e^T @ x_e (experts without rows give exact zeros)
    dw = grouped_gemm(dy, a, offs, mode=1)
    O.check_status()
    for e, c in enumerate(counts):
        ref = dy[o[e]: o[e] + c].float().t() @ a[o[e]: o[e] + c].float()
        if c:
            assert _rel(dw[e], ref) < 6e-3, e
        else:
            assert dw[e].abs().max().item() == 0


def test_expert_parallel_single_rank_matches_reference():
    torch.manual_seed(1)
    T, H, I, E, k = 512, 256, 128, 8, 2
    ws = MoEWorkspace(T, k, H, E, wait_s=5.0)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    router = torch.randn(T, E, device=DEV)
    idx, w, _ = topk_route(router, k)
    w = w.to(torch.bfloat16).requires_grad_()
    wgu = (torch.randn(E, 2 * I, H, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    wd = (torch.randn(E, H, I, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    for _ in range(2):  # second pass exercises buffer reuse / epochs
        for t in (x, w, wgu, wd):
            t.grad = None
        y = expert_parallel_ffn(x, idx, w, wgu, wd, ws)
        g = torch.randn_like(y)
        y.backward(g)
        torch.cuda.synchronize()
        O.check_status()
        xr, wr, gur, dr = (t.detach().float().requires_grad_() for t in (x, w, wgu, wd))
        yr = expert_ffn_reference(xr, idx, wr, gur, dr)
        yr.backward(g.float())
        assert _rel(y, yr) < 1.5e-2
        assert _rel(x.grad, xr.grad) < 2e-2
        assert _rel(w.grad, wr.grad) < 2e-2
        assert _rel(wgu.grad, gur.grad) < 2e-2
        assert _rel(wd.grad, dr.grad) < 2e-2


def test_token_switch_dispatch_combine_have_gradients():
    """``TokenSwitch.dispatch`` / ``combine`` composed with a per-row expert function against the
    dense formula, forward and backward (tokens, expert output rows and routing weights)."""
    from tensorplay_b200.distributed._token_switch import TokenSwitch
    torch.manual_seed(0)
    T, H, E, k = 96, 256, 4, 2
    sw = TokenSwitch(E, k, H, T)
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    logits = torch.randn(T, E, device=DEV)
    scale = torch.linspace(0.5, 2.0, E, device=DEV)          # "expert e" multiplies its rows by scale[e]
    r = sw.create_routing(logits)
    r.topk_weight = r.topk_weight.to(torch.bfloat16).requires_grad_()
    rows = sw.dispatch(x, r)                                  # [cap, H], expert-sorted
    offs = r.offsets.tolist()
    per_row = torch.zeros(rows.shape[0], 1, device=DEV)
    for e in range(E):
        per_row[offs[e]: offs[e + 1]] = scale[e]
    y = sw.combine((rows.float() * per_row).to(torch.bfloat16), r)
    g = torch.randn_like(y)
    y.backward(g)
    O.check_status()
    xr = x.detach().float().requires_grad_()
    wr = r.topk_weight.detach().float().requires_grad_()
    ref = (xr[:, None, :] * scale[r.topk_idx][..., None] * wr[..., None]).sum(1)
    ref.backward(g.float())
    assert _rel(y, ref) < 2e-2
    assert _rel(x.grad, xr.grad) < 2e-2
    assert _rel(r.topk_weight.grad, wr.grad) < 2e-2
