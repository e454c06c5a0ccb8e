"""Flash attention forward/backward (tcgen05) against an fp32 PyTorch reference."""
import pytest
import torch

import tensorplay_b200.ops as O
from tensorplay_b200.ops.attention import attention_reference, flash_attention

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


CASES = [
    # B, Tq, Tk, Hq, Hkv, D, causal
    (1, 128, 128, 1, 1, 128, False),
    (1, 128, 128, 1, 1, 128, True),
    (2, 256, 256, 4, 2, 128, True),
    (1, 512, 512, 8, 2, 128, True),
    (2, 200, 200, 4, 4, 128, True),
    (1, 333, 333, 2, 1, 128, False),
    (1, 384, 384, 12, 12, 64, True),
    (1, 128, 384, 4, 1, 128, True),
    (1, 1024, 1024, 8, 2, 128, True),
]


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,D,causal", CASES)
def test_flash_forward(B, Tq, Tk, Hq, Hkv, D, causal):
    torch.manual_seed(0)
    q = torch.randn(B, Tq, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, Tk, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, Tk, Hkv, D, device=DEV, dtype=torch.bfloat16)
    o = flash_attention(q, k, v, causal=causal)
    O.check_status()
    ref = attention_reference(q.float(), k.float(), v.float(), causal)
    assert _rel(o, ref) < 1e-2


@pytest.mark.parametrize("B,Tq,Tk,Hq,Hkv,D,causal", CASES)
def test_flash_backward(B, Tq, Tk, Hq, Hkv, D, causal):
    torch.manual_seed(1)
    q = torch.randn(B, Tq, Hq, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, Tk, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, Tk, Hkv, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    o = flash_attention(q, k, v, causal=causal)
    g = torch.randn_like(o)
    o.backward(g)
    O.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, causal)
    ref.backward(g.float())
    assert _rel(q.grad, qr.grad) < 2e-2
    assert _rel(k.grad, kr.grad) < 2e-2
    assert _rel(v.grad, vr.grad) < 2e-2


def test_flash_fused_qkv_strides():
    # q, k, v as slices of one projection buffer (the layout the model uses)
    torch.manual_seed(2)
    B, T, Hq, Hkv, D = 2, 256, 8, 2, 128
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, device=DEV, dtype=torch.bfloat16)
    q = qkv[..., : Hq * D].view(B, T, Hq, D)
    k = qkv[..., Hq * D: (Hq + Hkv) * D].view(B, T, Hkv, D)
    v = qkv[..., (Hq + Hkv) * D:].view(B, T, Hkv, D)
    o = flash_attention(q, k, v, causal=True)
    O.check_status()
    ref = attention_reference(q.float(), k.float(), v.float(), True)
    assert _rel(o, ref) < 1e-2


@pytest.mark.parametrize("n_splits", [1, 3, 8])
def test_decode_attention_device_length_and_split_kv(n_splits):
    """Decode form: few query rows per (batch, kv head), keys limited by a device-side length,
    optionally split over several CTAs and merged by LSE."""
    from tensorplay_b200.ops.attention import flash_fwd
    torch.manual_seed(5)
    B, G, Hkv, D, cap, used = 3, 4, 2, 128, 1024, 700
    q = torch.randn(B, G, Hkv, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, cap, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, cap, Hkv, D, device=DEV, dtype=torch.bfloat16)
    kv_len = torch.tensor([used], device=DEV, dtype=torch.int32)
    o, lse = flash_fwd(q, k, v, False, 1.0 / D ** 0.5, kv_len=kv_len, n_splits=n_splits)
    O.check_status()
    ref = attention_reference(q.float(), k[:, :used].float(), v[:, :used].float(), False)
    assert _rel(o, ref) < 1e-2
    s = torch.einsum("bghd,bthd->bhgt", q.float(), k[:, :used].float()) / D ** 0.5
    torch.testing.assert_close(lse[:, :, :G], torch.logsumexp(s, -1), rtol=1e-2, atol=2e-2)
