"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""
import pytest
import torch

import tensorplay_b200.ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (384, 200, 136), (1000, 328, 72),
                                   (4096, 1024, 512), (130, 6144, 4096)])
def test_gemm_layouts(a_mn, b_mn, M, N, K):
    torch.manual_seed(0)
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    if b_mn and N % 8:
        pytest.skip("MN-major B needs N % 8 == 0")
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    out = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
    O.check_status()
    assert out.shape == (M, N)
    assert _rel(out, ref) < 5e-3
    out32 = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert _rel(out32, ref) < 1e-4


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (384, 200, 136), (1000, 328, 72),
                                   (8192, 4096, 1024), (2048, 2304, 4096 + 8)])
@pytest.mark.parametrize("block_n", [256, 128])
def test_gemm_cta_pair(a_mn, b_mn, M, N, K, block_n):
    """The cta_group::2 kernel: 256-row tiles computed by two CTAs, each staging half of B."""
    from tensorplay_b200.ops._common import lib
    torch.manual_seed(3)
    lib().tpb_gemm_pair_block_n(block_n)
    try:
        _check_gemm_cta_pair(a_mn, b_mn, M, N, K)
    finally:
        lib().tpb_gemm_pair_block_n(0)


def _check_gemm_cta_pair(a_mn, b_mn, M, N, K):
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a leading dimension that is a multiple of 8")
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    out32 = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, impl="pair")
    O.check_status()
    assert _rel(out32, ref) < 1e-4
    bias = torch.randn(N, device=DEV, dtype=torch.float32)
    out = torch.ones(M, N, device=DEV, dtype=torch.bfloat16)
    O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out=out, bias=bias, accumulate=True, alpha=0.5, impl="pair")
    O.check_status()
    assert _rel(out, 0.5 * ref + bias + 1.0) < 5e-3


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (512, 1024, 8192), (4096, 6144, 2048), (1280, 2304, 1024 + 64)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
def test_gemm_cta_pair_split_tail(M, N, K, a_mn, b_mn):
    """CTA-pair kernel with the last wave split along K: same result as the unsplit run, call after call."""
    from tensorplay_b200.ops.gemm import enable_splitk
    torch.manual_seed(6)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    enable_splitk(enable=False)
    base = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, impl="pair")
    enable_splitk()
    try:
        for _ in range(3):  # flags must re-arm between calls
            out = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, impl="pair")
            O.check_status()
            assert _rel(out, base) < 2e-5
        outb = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, impl="pair")
        assert _rel(outb, a.float() @ b.float().t()) < 5e-3
    finally:
        enable_splitk(enable=False)


def test_gemm_bias_accumulate_alpha():
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    c0 = torch.randn(M, N, device=DEV, dtype=torch.float32)
    ref = 0.5 * (a.float() @ b.float().t()) + bias.float() + c0
    out = c0.clone()
    O.gemm(a, b, out=out, bias=bias, accumulate=True, alpha=0.5)
    O.check_status()
    assert _rel(out, ref) < 1e-4


def test_gemm_many_tiles_persistent():
    # more tiles than SMs: exercises the persistent loop, both TMEM stages and phase wrap
    torch.manual_seed(2)
    M, N, K = 8192, 4096, 1024
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    out = O.gemm(a, b)
    O.check_status()
    ref = a.float() @ b.float().t()
    assert _rel(out, ref) < 5e-3


@pytest.mark.parametrize("M,N,K", [(4096, 4096, 4096), (512, 1024, 8192), (4096, 6144, 2048), (1152, 2304, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True)])
def test_gemm_splitk_tail(M, N, K, a_mn, b_mn):
    """The last partial wave is split along K over idle SMs; results must match the unsplit run."""
    from tensorplay_b200.ops.gemm import enable_splitk
    torch.manual_seed(5)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    A = a.t().contiguous() if a_mn else a
    B = b.t().contiguous() if b_mn else b
    enable_splitk(enable=False)
    base = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    enable_splitk()
    try:
        for _ in range(3):  # flags must re-arm between calls
            out = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
            O.check_status()
            assert _rel(out, base) < 2e-5
        outb = O.gemm(A, B, a_mn=a_mn, b_mn=b_mn)
        assert _rel(outb, a.float() @ b.float().t()) < 5e-3
    finally:
        enable_splitk(enable=False)


@pytest.mark.parametrize("M,N,K", [(64, 1280, 8192), (64, 8192, 1024), (64, 7168, 8192), (100, 1000, 3584),
                                   (8, 8192, 3584), (130, 520, 2048)])
def test_gemm_few_rows_split_with_distributed_reduction(M, N, K):
    """Decode-sized products: every tile is split along K, each split parks its partial rows and reduces a
    column slice of the tile. Plain, biased, scaled and accumulating epilogues; flags re-arm between calls."""
    from tensorplay_b200.ops.gemm import enable_splitk
    torch.manual_seed(11)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.float32)
    ref = a.float() @ b.float().t()
    enable_splitk()
    try:
        outs = [O.gemm(a, b, out_dtype=torch.float32, impl="single") for _ in range(12)]  # back to back
        O.check_status()
        for out32 in outs:
            assert _rel(out32, ref) < 2e-5
        out = O.gemm(a, b, impl="single")
        assert _rel(out, ref) < 5e-3
        acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
        O.gemm(a, b, out=acc, bias=bias, accumulate=True, alpha=0.5, impl="single")
        O.check_status()
        assert _rel(acc, 0.5 * ref + bias + 1.0) < 2e-5
        accb = torch.ones(M, N, device=DEV, dtype=torch.bfloat16)
        O.gemm(a, b, out=accb, bias=bias, accumulate=True, alpha=0.5, impl="single")
        O.check_status()
        assert _rel(accb, 0.5 * ref + bias + 1.0) < 5e-3
    finally:
        enable_splitk(enable=False)


def test_linear_autograd():
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    bias = torch.randn(384, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = O.linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 5e-3
    assert _rel(x.grad, xr.grad) < 5e-3
    assert _rel(w.grad, wr.grad) < 5e-3
    assert _rel(bias.grad, br.grad) < 1e-2


@pytest.mark.parametrize("rows,H", [(7, 128), (300, 768), (513, 2048), (1024, 4096), (64, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, H, with_res):
    torch.manual_seed(4)
    x = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    res = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_res else None
    out = O.rms_norm(x, w, 1e-5, res)
    y, r = out if with_res else (out, None)
    g = torch.randn_like(y)
    gr = torch.randn_like(y) if with_res else None
    (y.float() * g.float()).sum().backward() if not with_res else \
        ((y.float() * g.float()).sum() + (r.float() * gr.float()).sum()).backward()
    xr = x.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if with_res else None
    h = xr + rr if with_res else xr
    if with_res:
        h = h.detach().to(torch.bfloat16).float() + (h - h.detach())  # stream rounded to bf16, straight-through
    yr = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    loss = (yr * g.float()).sum()
    if with_res:
        loss = loss + (h * gr.float()).sum()
    loss.backward()
    assert _rel(y, yr) < 8e-3
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    if with_res:
        assert _rel(res.grad, rr.grad) < 1e-2


@pytest.mark.parametrize("rows,H", [(33, 768), (2048, 1024)])
def test_layernorm(rows, H):
    torch.manual_seed(5)
    x = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    b = (0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = O.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (H,), wr, br, 1e-5)
    yr.backward(g.float())
    assert _rel(y, yr) < 8e-3
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    assert _rel(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope(interleaved):
    torch.manual_seed(6)
    B, T, H, D = 2, 37, 6, 128
    x = torch.randn(B, T, H, D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    cos, sin = O.rope_tables(64, D, 500000.0, device=DEV)
    pos = torch.randint(0, 64, (B, T), device=DEV)
    from tensorplay_b200.ops.rope import _rope_ref
    for p in (None, pos):
        x.grad = None
        y = O.apply_rope(x * 1.0, cos, sin, p, interleaved)
        g = torch.randn_like(y)
        y.backward(g)
        xr = x.detach().float().requires_grad_()
        yr = _rope_ref(xr, cos, sin, p, interleaved, 1.0)
        yr.backward(g.float())
        assert _rel(y, yr) < 8e-3
        assert _rel(x.grad, xr.grad) < 8e-3


def test_rope_from_a_strided_source_and_in_place():
    """The q/k heads of a packed QKV projection are rotated straight out of the packed buffer; the in-place
    form gives the same values."""
    torch.manual_seed(8)
    B, T, Hq, Hkv, D = 2, 33, 8, 2, 128
    packed = torch.randn(B, T, Hq + 2 * Hkv, D, device=DEV, dtype=torch.bfloat16)
    cos, sin = O.rope_tables(64, D, 500000.0, device=DEV)
    from tensorplay_b200.ops.rope import _rope_ref
    src = packed[:, :, : Hq + Hkv]
    keep = packed.clone()
    want = _rope_ref(src.float(), cos, sin, None, False, 1.0)
    out = O.apply_rope(src, cos, sin)
    assert out.is_contiguous() and torch.equal(packed, keep)          # the source is untouched
    assert _rel(out, want) < 8e-3
    inpl = src.contiguous()
    O.apply_rope(inpl, cos, sin, inplace=True)
    assert torch.equal(inpl, out)
    # gradient through the strided source
    pk = packed.clone().requires_grad_(True)
    y = O.apply_rope(pk[:, :, : Hq + Hkv], cos, sin)
    g = torch.randn_like(y)
    y.backward(g)
    pr = packed.float().requires_grad_(True)
    _rope_ref(pr[:, :, : Hq + Hkv], cos, sin, None, False, 1.0).backward(g.float())
    assert _rel(pk.grad, pr.grad) < 8e-3
    O.check_status()


def test_swiglu_gelu():
    torch.manual_seed(7)
    gu = torch.randn(129, 2 * 1408, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = O.swiglu_packed(gu)
    g = torch.randn_like(y)
    y.backward(g)
    gr = gu.detach().float().requires_grad_()
    yr = torch.nn.functional.silu(gr[:, :1408]) * gr[:, 1408:]
    yr.backward(g.float())
    assert _rel(y, yr) < 8e-3 and _rel(gu.grad, gr.grad) < 1e-2
    for approx in ("none", "tanh"):
        x = torch.randn(77, 3072, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        y = O.gelu(x, approx)
        g = torch.randn_like(y)
        y.backward(g)
        xr = x.detach().float().requires_grad_()
        yr = torch.nn.functional.gelu(xr, approximate=approx)
        yr.backward(g.float())
        assert _rel(y, yr) < 8e-3 and _rel(x.grad, xr.grad) < 1e-2


@pytest.mark.parametrize("V", [512, 50257, 128256])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_cross_entropy(V, reduction):
    torch.manual_seed(8)
    rows = 96
    Vp = (V + 7) // 8 * 8
    buf = torch.randn(rows, Vp, device=DEV, dtype=torch.bfloat16) * 2
    logits = buf[:, :V].detach().requires_grad_()
    tgt = torch.randint(0, V, (rows,), device=DEV)
    tgt[5] = -100
    ref_in = logits.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(ref_in, tgt, reduction=reduction)
    g = torch.randn_like(ref)
    ref.backward(g)
    loss = O.cross_entropy(logits, tgt, reduction=reduction)
    loss.backward(g.to(loss.dtype))
    assert _rel(loss, ref) < 2e-3
    assert _rel(logits.grad, ref_in.grad) < 1e-2


def test_adamw_flat_and_multi():
    torch.manual_seed(9)
    n = 100003
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master = p.clone()
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    model = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    for step in range(1, 4):
        gb = (g * step).to(torch.bfloat16)
        ref.grad = gb.float()
        opt.step()
        O.adamw_flat_(master, m, v, gb, model, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                      weight_decay=0.1, step=step)
    assert torch.allclose(master, ref.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(model, master.to(torch.bfloat16))
    # multi-tensor
    sizes = [5, 70000, 131072, 33, 200001]
    ps = [torch.randn(s, device=DEV) for s in sizes]
    gs = [torch.randn(s, device=DEV) for s in sizes]
    refs = [torch.nn.Parameter(t.clone()) for t in ps]
    opt = torch.optim.AdamW(refs, lr=3e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    ms = [torch.zeros_like(t) for t in ps]
    vs = [torch.zeros_like(t) for t in ps]
    for r, gg in zip(refs, gs):
        r.grad = gg.clone()
    opt.step()
    O.adamw_multi_(ps, ms, vs, gs, None, lr=3e-3, beta1=0.9, beta2=0.999, eps=1e-8,
                   weight_decay=0.01, step=1)
    for a, b in zip(ps, refs):
        assert torch.allclose(a, b.detach(), rtol=1e-5, atol=1e-6)
    ss = torch.zeros(1, device=DEV)
    for gg in gs:
        O.sumsq_(gg, ss)
    tot = sum((gg.double() ** 2).sum() for gg in gs)
    assert abs(ss.item() - tot.item()) / tot.item() < 1e-4


def test_nvtx_ranges_inside_the_kernel_library():
    """With ``profiler.nvtx_kernels()`` the launching entry points push an NVTX range each; results are the
    same and the switch goes back to its previous state."""
    from tensorplay_b200 import profiler
    from tensorplay_b200.ops._common import lib
    a = torch.randn(512, 256, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.ones(256, device=DEV, dtype=torch.bfloat16)
    plain = O.gemm(a, b), O.rms_norm(a, w)
    assert lib().tpb_nvtx_enabled() == 0
    with profiler.nvtx_kernels():
        assert lib().tpb_nvtx_enabled() == 1
        ranged = O.gemm(a, b), O.rms_norm(a, w)
    assert lib().tpb_nvtx_enabled() == 0
    O.check_status()
    for x, y in zip(plain, ranged):
        assert torch.equal(x, y)


def test_flop_counter_sees_native_kernels():
    from tensorplay_b200.utils.flop_counter import FlopCounterMode
    M, N, K = 256, 384, 128
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(N, K, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    B, T, H, D = 1, 256, 2, 128
    q, k, v = (torch.randn(B, T, H, D, device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    with FlopCounterMode(display=False) as fc:
        O.linear(a, w).float().sum().backward()                 # forward + dgrad + wgrad
        O.flash_attention(q, k, v, causal=True).float().sum().backward()
    c = fc.get_flop_counts()["Global"]
    assert c["tpb.gemm"] == 3 * 2 * M * N * K
    assert c["tpb.flash_attention_forward"] == 4 * B * H * T * T * D // 2
    assert c["tpb.flash_attention_backward"] == 10 * B * H * T * T * D // 2
