"""The CPU (oracle) paths of the core ops against plain formulas written out here: these paths are
what every GPU numerics test is compared with, so they get their own independent check."""
import math

import torch

from tensorplay_b200 import ops


def test_rms_norm_with_residual_and_layer_norm():
    g = torch.Generator().manual_seed(0)
    x, r, w = torch.randn(5, 16, generator=g), torch.randn(5, 16, generator=g), torch.rand(16, generator=g) + 0.5
    y = ops.rms_norm(x, w, 1e-5)
    torch.testing.assert_close(y, x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * w)
    y2, s = ops.rms_norm(x, w, 1e-5, residual=r)
    h = x + r
    torch.testing.assert_close(s, h)
    torch.testing.assert_close(y2, h / torch.sqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * w)
    b = torch.randn(16, generator=g)
    torch.testing.assert_close(ops.layer_norm(x, w, b, 1e-5), torch.nn.functional.layer_norm(x, (16,), w, b, 1e-5))


def test_rope_tables_and_rotation():
    cos, sin = ops.rope_tables(32, 8, 10000.0)
    assert cos.shape[0] == 32
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2, 6, 3, 8, generator=g)
    y = ops.apply_rope(x, cos, sin)
    # NeoX layout: pairs (i, i + D/2) rotate by pos * theta^(-2i/D)
    inv = 10000.0 ** (-torch.arange(0, 4).float() * 2 / 8)
    ang = torch.arange(6).float()[:, None] * inv[None, :]
    c, s = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    x1, x2 = x[..., :4], x[..., 4:]
    torch.testing.assert_close(y, torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), -1), rtol=1e-5, atol=1e-5)
    # explicit positions: rotating position p equals slicing the table at p; norms are preserved
    pos = torch.tensor([[3, 3, 7, 0, 1, 2], [0, 1, 2, 3, 4, 5]])
    yp = ops.apply_rope(x, cos, sin, pos)
    torch.testing.assert_close(yp[1], y[1])
    torch.testing.assert_close(yp.norm(dim=-1), x.norm(dim=-1), rtol=1e-5, atol=1e-5)
    yi = ops.apply_rope(x, cos, sin, None, interleaved=True)
    xe, xo = x[..., 0::2], x[..., 1::2]
    torch.testing.assert_close(yi[..., 0::2], xe * c - xo * s, rtol=1e-5, atol=1e-5)


def test_swiglu_and_cross_entropy():
    g = torch.Generator().manual_seed(2)
    a, b = torch.randn(4, 10, generator=g), torch.randn(4, 10, generator=g)
    torch.testing.assert_close(ops.swiglu(a, b), torch.nn.functional.silu(a) * b)
    torch.testing.assert_close(ops.swiglu_packed(torch.cat((a, b), -1)), torch.nn.functional.silu(a) * b)
    logits = torch.randn(7, 12, generator=g, requires_grad=True)
    t = torch.tensor([1, 5, -100, 0, 11, -100, 3])
    l = ops.cross_entropy(logits, t)
    ref = torch.nn.functional.cross_entropy(logits, t, ignore_index=-100)
    torch.testing.assert_close(l, ref)
    l.backward()
    assert logits.grad[2].abs().sum() == 0 and logits.grad[0].abs().sum() > 0
    torch.testing.assert_close(ops.cross_entropy(logits.detach(), t, reduction="sum"),
                               torch.nn.functional.cross_entropy(logits.detach(), t, reduction="sum"))


def test_gemm_layout_flags_bias_and_accumulate():
    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(6, 10, generator=g), torch.randn(4, 10, generator=g)
    ref = a @ b.t()
    f32 = dict(out_dtype=torch.float32)
    torch.testing.assert_close(ops.gemm(a, b, **f32), ref)
    torch.testing.assert_close(ops.gemm(a.t().contiguous(), b, a_mn=True, **f32), ref)
    torch.testing.assert_close(ops.gemm(a, b.t().contiguous(), b_mn=True, **f32), ref)
    bias = torch.randn(4, generator=g)
    torch.testing.assert_close(ops.gemm(a, b, bias=bias, alpha=0.5, **f32), 0.5 * ref + bias)
    out = torch.ones(6, 4)
    ops.gemm(a, b, out=out, accumulate=True)
    torch.testing.assert_close(out, ref + 1)
    torch.testing.assert_close(ops.linear(a.view(2, 3, 10), b, bias), (ref + bias).view(2, 3, 4))


def test_attention_reference_gqa_and_bottom_right_causal():
    g = torch.Generator().manual_seed(4)
    B, Tq, Tk, Hq, Hkv, D = 2, 3, 5, 4, 2, 8
    q, k, v = (torch.randn(B, t, h, D, generator=g) for t, h in ((Tq, Hq), (Tk, Hkv), (Tk, Hkv)))
    o = ops.flash_attention(q, k, v, causal=True)
    ref = torch.zeros_like(o)
    for b in range(B):
        for h in range(Hq):
            kh = h // (Hq // Hkv)
            s = (q[b, :, h] @ k[b, :, kh].t()) / math.sqrt(D)
            # the last query is aligned with the last key: query i sees keys j <= i + (Tk - Tq)
            mask = torch.arange(Tk)[None, :] > (torch.arange(Tq)[:, None] + (Tk - Tq))
            ref[b, :, h] = torch.softmax(s.masked_fill(mask, float("-inf")), -1) @ v[b, :, kh]
    torch.testing.assert_close(o, ref, rtol=1e-5, atol=1e-5)
    # packed projection + RoPE path equals the unpacked calls
    T = 6
    qkv = torch.randn(B, T, (Hq + 2 * Hkv) * D, generator=g)
    cos, sin = ops.rope_tables(T, D)
    p = qkv.view(B, T, Hq + 2 * Hkv, D)
    want = ops.flash_attention(ops.apply_rope(p[:, :, :Hq], cos, sin), ops.apply_rope(p[:, :, Hq:Hq + Hkv], cos, sin),
                               p[:, :, Hq + Hkv:], causal=True).reshape(B, T, Hq * D)
    torch.testing.assert_close(ops.qkv_attention(qkv, cos, sin, None, Hq, Hkv, D), want, rtol=1e-5, atol=1e-5)


def test_adamw_flat_matches_torch_adamw_and_clipping_helpers():
    g = torch.Generator().manual_seed(5)
    p0 = torch.randn(50, generator=g)
    ref = torch.nn.Parameter(p0.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master, m, v = p0.clone(), torch.zeros(50), torch.zeros(50)
    model = torch.zeros(50, dtype=torch.bfloat16)
    for step in range(1, 4):
        grad = torch.randn(50, generator=g)
        ref.grad = grad.clone()
        opt.step()
        ops.adamw_flat_(master, m, v, grad, model, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    torch.testing.assert_close(master, ref.detach(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(model.float(), master.bfloat16().float())
    acc, coef = torch.zeros(1), torch.zeros(1)
    x = torch.randn(100, generator=g)
    ops.sumsq_(x, acc)
    torch.testing.assert_close(acc, x.pow(2).sum().view(1))
    ops.clip_coef_(acc, 1.0, coef)
    torch.testing.assert_close(coef, (1.0 / (x.norm() + 1e-6)).clamp(max=1.0).view(1), rtol=1e-4, atol=1e-6)
