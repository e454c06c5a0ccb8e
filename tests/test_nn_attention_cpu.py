"""``nn.attention``: backend selection, the flash-implementation registry and variable-length
attention against per-sequence dense attention (CPU: the fp32 formula serves every sequence)."""
import pytest
import torch

import tensorplay_b200 as tp
from tensorplay_b200.nn import attention as A
from tensorplay_b200.nn import functional as F
from tensorplay_b200.nn.attention import AuxRequest, SDPBackend, sdpa_kernel, varlen_attn


def test_own_submodules_are_not_shadowed_by_torch():
    assert tp.nn.functional.__name__ == "tensorplay_b200.nn.functional"
    assert tp.nn.attention.__name__ == "tensorplay_b200.nn.attention"
    assert tp.nn.parallel.__name__ == "tensorplay_b200.nn.parallel"
    assert A.causal_lower_right is torch.nn.attention.bias.causal_lower_right


def test_sdpa_kernel_selects_and_restores():
    torch.manual_seed(0)
    q, k = torch.randn(2, 4, 16, 32), torch.randn(2, 2, 16, 32)
    v = torch.randn(2, 2, 16, 32)
    base = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    with sdpa_kernel(SDPBackend.MATH):
        assert A._cur_sdpa_kernel_backends() == [SDPBackend.MATH]
        assert torch.allclose(F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True), base, atol=1e-6)
    with sdpa_kernel([SDPBackend.MATH, SDPBackend.FLASH_ATTENTION]):
        assert A._cur_sdpa_kernel_backends() == [SDPBackend.FLASH_ATTENTION, SDPBackend.MATH]   # default order
    with sdpa_kernel([SDPBackend.MATH, SDPBackend.FLASH_ATTENTION], set_priority=True):
        assert A._cur_sdpa_kernel_backends() == [SDPBackend.MATH, SDPBackend.FLASH_ATTENTION]
    with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
        with pytest.raises(RuntimeError, match="No available kernel"):
            F.scaled_dot_product_attention(q, k, v)   # fp32 on the CPU: the flash kernels cannot take it
    assert len(A._cur_sdpa_kernel_backends()) == 4
    with pytest.raises(AssertionError):
        with sdpa_kernel("flash"):
            pass


def test_flash_impl_registry():
    calls = []

    def fake(q, k, v, causal, scale):
        calls.append((tuple(q.shape), causal))
        return torch.zeros_like(q)

    A.register_flash_attention_impl("fake", fake)
    assert "fake" in A.list_flash_attention_impls() and A.current_flash_attention_impl() == "tcgen05"
    A.activate_flash_attention_impl("fake")
    try:
        q = torch.randn(6, 2, 8)
        cu = torch.tensor([0, 6], dtype=torch.int32)
        out = A._flash(q[None], q[None], q[None], True, 1.0)
        assert calls == [((1, 6, 2, 8), True)] and out.abs().sum() == 0
    finally:
        A.restore_flash_attention_impl()
    assert A.current_flash_attention_impl() == "tcgen05"
    with pytest.raises(KeyError):
        A.activate_flash_attention_impl("missing")


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_attention_matches_per_sequence_attention(causal):
    torch.manual_seed(1)
    lens_q, lens_k = [5, 9, 3, 0, 7], [5, 12, 3, 4, 7]
    cq = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    ck = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    Q = torch.randn(int(cq[-1]), 4, 32, requires_grad=True)
    K = torch.randn(int(ck[-1]), 2, 32, requires_grad=True)
    V = torch.randn(int(ck[-1]), 2, 32, requires_grad=True)
    out, lse = varlen_attn(Q, K, V, cq, ck, max(lens_q), max(lens_k), is_causal=causal, return_aux=AuxRequest(lse=True))
    ref = []
    for i in range(len(lens_q)):
        if lens_q[i] == 0:
            continue
        q, k, v = Q[cq[i]:cq[i + 1]], K[ck[i]:ck[i + 1]], V[ck[i]:ck[i + 1]]
        ref.append(F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                                                  is_causal=causal, enable_gqa=True)[0].transpose(0, 1))
    ref = torch.cat(ref)
    assert torch.allclose(out, ref, atol=1e-5)
    assert lse.shape == (4, int(cq[-1]))
    g = torch.randn_like(out)
    gq, gk = torch.autograd.grad(out, (Q, K), g, retain_graph=True)
    rq, rk = torch.autograd.grad(ref, (Q, K), g)
    assert torch.allclose(gq, rq, atol=1e-5) and torch.allclose(gk, rk, atol=1e-5)
    # a window of two keys to the left: every row sees at most three keys
    w = varlen_attn(Q, K, V, cq, ck, max(lens_q), max(lens_k), is_causal=True, window_size=(2, 0))
    q0, k0, v0 = Q[:5], K[:5], V[:5]
    s = torch.einsum("qhd,khd->hqk", q0, k0.repeat_interleave(2, 1)) / 32 ** 0.5
    i, j = torch.arange(5).view(-1, 1), torch.arange(5).view(1, -1)
    s = s.masked_fill(~((j <= i) & (j >= i - 2)), float("-inf"))
    want = torch.einsum("hqk,khd->qhd", s.softmax(-1), v0.repeat_interleave(2, 1))
    assert torch.allclose(w[:5], want, atol=1e-5)
    with pytest.raises(ValueError):
        varlen_attn(Q, K, V, cq, ck, 2, 2)
