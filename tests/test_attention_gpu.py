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


def _close(a, b, tol):
    """Relative error in norm, or both negligibly small (a window of one key has exactly zero dq and dk)."""
    return _rel(a, b) < tol or (a.float() - b.float()).abs().max().item() < 1e-4


def _fwd_bwd(q, k, v, **kw):
    q = q.clone().requires_grad_(True)
    k = k.clone().requires_grad_(True)
    v = v.clone().requires_grad_(True)
    o = flash_attention(q, k, v, **kw)
    g = torch.Generator(device="cpu").manual_seed(9)
    do = torch.randn(o.shape, generator=g).to(o.device, o.dtype)
    o.backward(do)
    return o, q.grad, k.grad, v.grad


@pytest.mark.parametrize("T,window", [(512, 128), (1000, 200), (1024, 64), (777, 1), (640, 4096)])
@pytest.mark.parametrize("D", [128, 64])
def test_flash_sliding_window(T, window, D):
    """Causal local attention inside the kernels: KV blocks left of the window are skipped, the blocks on
    its edge are masked; forward and all three gradients against the fp32 formula."""
    torch.manual_seed(4)
    B, Hq, Hkv = 2, 4, 2
    q = torch.randn(B, T, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, device=DEV, dtype=torch.bfloat16)
    o, dq, dk, dv = _fwd_bwd(q, k, v, causal=True, window=window)
    O.check_status()
    ro, rq, rk, rv = _fwd_bwd(q.float(), k.float(), v.float(), causal=True, window=window)
    assert _rel(o, ro) < 1e-2
    assert _close(dq, rq, 2e-2) and _close(dk, rk, 2e-2) and _close(dv, rv, 2e-2)


@pytest.mark.parametrize("lens", [[128, 128], [100, 300, 57], [1, 255, 640, 3], [513], [64, 64, 64, 64, 700]])
@pytest.mark.parametrize("causal", [True, False])
def test_flash_packed_sequences(lens, causal):
    """Several sequences packed into one row: every token attends only inside its own sequence (bounds per
    token), equal to running the sequences one by one."""
    from tensorplay_b200.ops.attention import segment_bounds
    torch.manual_seed(5)
    Hq, Hkv, D = 4, 2, 128
    total = sum(lens)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    q = torch.randn(1, total, Hq, D, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(1, total, Hkv, D, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(1, total, Hkv, D, device=DEV, dtype=torch.bfloat16)
    ss, se = segment_bounds(cu, total)
    assert ss.tolist()[: lens[0]] == [0] * lens[0] and se.tolist()[-1] == total
    o, dq, dk, dv = _fwd_bwd(q, k, v, causal=causal, seg_start=ss.view(1, -1), seg_end=se.view(1, -1))
    O.check_status()
    # oracle: sequence by sequence with the dense fp32 formula
    outs, gq, gk, gv = [], [], [], []
    g = torch.Generator(device="cpu").manual_seed(9)
    do = torch.randn(o.shape, generator=g).to(DEV).float()
    a = 0
    for n in lens:
        qs = q[:, a:a + n].float().requires_grad_(True)
        ks = k[:, a:a + n].float().requires_grad_(True)
        vs = v[:, a:a + n].float().requires_grad_(True)
        os_ = attention_reference(qs, ks, vs, causal)
        os_.backward(do[:, a:a + n])
        outs.append(os_.detach()); gq.append(qs.grad); gk.append(ks.grad); gv.append(vs.grad)
        a += n
    assert _rel(o, torch.cat(outs, 1)) < 1e-2
    assert _rel(dq, torch.cat(gq, 1)) < 2e-2
    assert _rel(dk, torch.cat(gk, 1)) < 2e-2
    assert _rel(dv, torch.cat(gv, 1)) < 2e-2


def test_varlen_attn_single_launch_matches_per_sequence():
    from tensorplay_b200.nn.attention import varlen_attn
    torch.manual_seed(6)
    lens = [200, 56, 300]
    total = sum(lens)
    cu = torch.tensor([0, 200, 256, 556], device=DEV, dtype=torch.int32)
    q = torch.randn(total, 4, 128, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(total, 2, 128, device=DEV, dtype=torch.bfloat16)
    v = torch.randn(total, 2, 128, device=DEV, dtype=torch.bfloat16)
    o = varlen_attn(q, k, v, cu, cu, 300, 300, is_causal=True)
    ow = varlen_attn(q, k, v, cu, cu, 300, 300, is_causal=True, window_size=(31, 0))
    O.check_status()
    a = 0
    for n in lens:
        ref = attention_reference(q[None, a:a + n].float(), k[None, a:a + n].float(), v[None, a:a + n].float(), True)[0]
        refw = attention_reference(q[None, a:a + n].float(), k[None, a:a + n].float(), v[None, a:a + n].float(), True,
                                   window=32)[0]
        assert _rel(o[a:a + n], ref) < 1e-2
        assert _rel(ow[a:a + n], refw) < 1e-2
        a += n


@pytest.mark.parametrize("D,Hq,Hkv", [(96, 4, 2), (256, 2, 2), (32, 8, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_head_dims_without_a_kernel_use_library_attention(D, Hq, Hkv, causal):
    """Head dims other than 64 / 128 run through PyTorch's attention (no score matrix in memory) with the same
    semantics: grouped heads, causal or full, gradients."""
    from tensorplay_b200.ops.attention import attention_reference, flash_attention
    torch.manual_seed(0)
    B, T = 2, 200
    q = torch.randn(B, T, Hq, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, T, Hkv, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    o = flash_attention(q, k, v, causal=causal)
    g = torch.randn_like(o)
    o.backward(g)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = attention_reference(qr, kr, vr, causal, D ** -0.5)
    ref.backward(g.float())
    assert o.shape == (B, T, Hq, D) and (o.float() - ref).abs().max() < 0.03
    for a, b in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (a.float() - b).abs().max() < 0.05 * max(1.0, b.abs().max().item())

