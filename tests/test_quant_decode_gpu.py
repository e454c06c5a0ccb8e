"""Quantised GEMM / GEMV, quantise-dequantise, embedding, KV-cache append and sampling kernels
against plain PyTorch fp32 references of the same ops."""
import pytest
import torch

import tensorplay_b200.ops as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 520, 1040), (1024, 4096, 4096), (5, 24, 48)])
def test_int8_gemm_matches_integer_reference(M, N, K):
    torch.manual_seed(0)
    a = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=DEV)
    w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=DEV)
    sa = torch.rand(M, device=DEV) * 0.01 + 0.001
    sw = torch.rand(N, device=DEV) * 0.01 + 0.001
    bias = torch.randn(N, device=DEV).bfloat16()
    y = O.int8_gemm(a, w, sa, sw, bias)
    O.check_status()
    ref = (a.double() @ w.double().t()).float() * sa[:, None] * sw[None, :] + bias.float()
    torch.testing.assert_close(y.float(), ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item())
    # exact integer accumulation: unit scales, small values
    y1 = O.int8_gemm(a.clamp(-3, 3), w.clamp(-3, 3))
    ref1 = (a.clamp(-3, 3).float() @ w.clamp(-3, 3).float().t())
    torch.testing.assert_close(y1.float(), ref1.bfloat16().float())


def test_int8_rowwise_quantise():
    x = (torch.randn(257, 1024, device=DEV) * 3).bfloat16()
    x[5] = 0
    q, s = O.quantize_int8_rowwise(x)
    qr, sr = O.quantize_int8_rowwise(x.cpu())
    torch.testing.assert_close(s.cpu(), sr)
    assert (q.cpu().int() - qr.int()).abs().max() <= 1
    assert (q.cpu() != qr).float().mean() < 1e-3


@pytest.mark.parametrize("bits,group,K", [(8, 0, 2048), (8, 128, 2048), (4, 128, 2048), (4, 64, 2048),
                                          (8, 16, 2048),   # one group per lane slice of the MMA kernel
                                          (8, 0, 2064), (4, 16, 2064)])  # K off the MMA chunk: CUDA-core kernel
@pytest.mark.parametrize("M", [1, 3, 16])
@pytest.mark.parametrize("version,fold", [(1, True), (2, True), (2, False)])
def test_weight_only_gemv(bits, group, K, M, version, fold):
    """Both versions of the warp-MMA kernel (2 = the loop written for instruction count), the second with scale
    and zero point applied per 128-k chunk (4 bits, groups >= 128: the default) or per weight."""
    from tensorplay_b200.ops.quant import gemv_config
    gemv_config(0, False, version, fold)
    try:
        _check_weight_only_gemv(bits, group, K, M)
    finally:
        gemv_config(0, False, 2)


@pytest.mark.parametrize("group,K", [(128, 4096), (256, 4096), (512, 2048)])
def test_w4a16_chunk_scaling_keeps_the_accuracy_with_biased_activations(group, K):
    """Activations with a large common offset make the 128 * sum(x) term of the chunk-scaled form large; the
    result must still sit within bf16 output rounding of the per-weight form and of the fp32 oracle."""
    from tensorplay_b200.ops.quant import gemv_config
    torch.manual_seed(2)
    N, M = 520, 5
    w = torch.randn(N, K, device=DEV)
    x = (torch.rand(M, K, device=DEV) * 2 + 3).bfloat16()          # every element in [3, 5)
    q, s, z = O.quantize_weight_int4(w, group)
    wd = O.dequantize_weight(q, s, z, 4, group).float()
    ref = x.float() @ wd.t()
    try:
        gemv_config(0, False, 2, True)
        y_fold = O.weight_only_linear(x, q, s, z, None, 4, group).float()
        gemv_config(0, False, 2, False)
        y_each = O.weight_only_linear(x, q, s, z, None, 4, group).float()
    finally:
        gemv_config(0, False, 2)
    scale = ref.abs().max().item()
    assert (y_fold - ref).abs().max() <= 1.2 * (y_each - ref).abs().max() + 2e-3 * scale
    assert (y_fold - ref).abs().max() < 8e-3 * scale


def _check_weight_only_gemv(bits, group, K, M):
    torch.manual_seed(1)
    N = 1000
    w = torch.randn(N, K, device=DEV)
    x = torch.randn(M, K, device=DEV).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    if bits == 8:
        q, s = O.quantize_weight_int8(w, group)
        z = None
    else:
        q, s, z = O.quantize_weight_int4(w, group)
    y = O.weight_only_linear(x, q, s, z, bias, bits, group)
    wd = O.dequantize_weight(q.cpu(), s.cpu(), None if z is None else z.cpu(), bits, group).float()
    ref = x.float().cpu() @ wd.t() + bias.float().cpu()
    torch.testing.assert_close(y.float().cpu(), ref, rtol=2e-2, atol=0.6)  # bf16 output, |y| up to ~150
    # dequantise kernel = CPU expression, bit for bit
    torch.testing.assert_close(O.dequantize_weight(q, s, z, bits, group).cpu().float(), wd)
    # prefill path (dequantise + tensor-core GEMM)
    xl = torch.randn(64, K, device=DEV).bfloat16()
    yl = O.weight_only_linear(xl, q, s, z, bias, bits, group)
    torch.testing.assert_close(yl.float().cpu(), xl.float().cpu() @ wd.t() + bias.float().cpu(), rtol=2e-2, atol=0.5)


@pytest.mark.parametrize("dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("per_row", [False, True])
def test_fp8_quantise_dequantise(dtype, per_row):
    x = (torch.randn(64, 512, device=DEV) * 10).bfloat16()
    fmax = 448.0 if dtype == torch.float8_e4m3fn else 57344.0
    amax = x.float().abs().amax(dim=-1, keepdim=True) if per_row else x.float().abs().amax()
    scale = (amax / fmax).clamp(min=1e-12)
    q = O.fp8_quantize(x, scale, dtype)
    ref = (x.float().cpu() / scale.cpu()).clamp(-fmax, fmax).to(dtype)
    assert q.dtype == dtype
    torch.testing.assert_close(q.cpu().float(), ref.float())
    d = O.fp8_dequantize(q, scale)
    torch.testing.assert_close(d.cpu().float(), (ref.float() * scale.cpu()).bfloat16().float())


def test_embedding_forward_backward():
    torch.manual_seed(2)
    V, H = 1000, 256
    w = torch.randn(V, H, device=DEV).bfloat16().requires_grad_()
    ids = torch.randint(0, V, (4, 333), device=DEV)
    ids[0, :50] = 7  # heavy duplicates
    y = O.embedding(ids, w)
    torch.testing.assert_close(y, w.detach()[ids])
    g = torch.randn_like(y)
    y.backward(g)
    ref = torch.zeros(V, H).index_add_(0, ids.reshape(-1).cpu(), g.reshape(-1, H).float().cpu())
    torch.testing.assert_close(w.grad.float().cpu(), ref, rtol=2e-2, atol=0.5)  # bf16 accumulation of up to 50 duplicates
    # fp32 destination
    dw = torch.zeros(V, H, device=DEV)
    from tensorplay_b200.ops.decode import embedding_backward_
    embedding_backward_(dw, ids, g)
    torch.testing.assert_close(dw.cpu(), ref, rtol=1e-5, atol=1e-4)


def test_kv_append_contiguous_and_paged():
    B, H, S, D, T = 3, 4, 64, 128, 5
    cache = torch.zeros(B, H, S, D, device=DEV, dtype=torch.bfloat16)
    new = torch.randn(B, H, T, D, device=DEV).bfloat16()
    O.kv_append(cache, new, 10)
    assert torch.equal(cache[:, :, 10:15], new) and cache[:, :, :10].abs().sum() == 0 and cache[:, :, 15:].abs().sum() == 0
    pos = torch.tensor([0, 7, 59], device=DEV, dtype=torch.int32)
    cache.zero_()
    O.kv_append(cache, new.transpose(1, 2).contiguous().transpose(1, 2), pos)  # strided source
    for b, p0 in enumerate(pos.tolist()):
        assert torch.equal(cache[b, :, p0:p0 + T], new[b])
    bs, nb = 16, 12
    pool = torch.zeros(nb, H, bs, D, device=DEV, dtype=torch.bfloat16)
    table = torch.tensor([[3, 1, 11], [0, 5, 2], [7, 8, 9]], device=DEV, dtype=torch.int32)
    O.kv_append(pool, new, 14, block_table=table, block_size=bs)
    ref = O.kv_append(torch.zeros(nb, H, bs, D).bfloat16(), new.cpu(), 14, block_table=table.cpu(), block_size=bs)
    assert torch.equal(pool.cpu(), ref)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("top_k,top_p", [(0, 1.0), (50, 1.0), (0, 0.9), (40, 0.8), (1, 1.0)])
def test_sampling_matches_reference_draw(dtype, top_k, top_p):
    torch.manual_seed(3)
    rows, V = 64, 32000
    logits = (torch.randn(rows, V, device=DEV) * 2).to(dtype)
    u = torch.rand(rows, device=DEV)
    got = O.sample(logits, 0.7, top_k, top_p, uniform=u)
    ref = O.sample_reference(logits.cpu().double(), u.cpu().double(), 0.7, top_k, top_p)
    # fp32 prefix sums may move a draw that lands within rounding of a CDF edge to the neighbour
    assert (got.cpu() == ref).float().mean() >= 0.95
    x = logits.float().cpu() / 0.7
    # every draw lies in the reference support
    if top_k:
        kth = torch.topk(x, top_k, dim=-1).values[:, -1]
        assert (x[torch.arange(rows), got.cpu()] >= kth).all()
    if top_k == 1:
        assert torch.equal(x[torch.arange(rows), got.cpu()], x.amax(-1))  # ties at the maximum all qualify


def test_sampling_distribution():
    probs = torch.tensor([0.5, 0.25, 0.125, 0.125], device=DEV)
    logits = probs.log().repeat(20000, 1).contiguous()
    got = O.sample(logits, 1.0, 0, 1.0)
    freq = torch.bincount(got, minlength=4).float() / got.numel()
    torch.testing.assert_close(freq, probs, atol=0.02, rtol=0)
    got = O.sample(logits, 1.0, 0, 0.7)  # nucleus keeps {0.5, 0.25}
    freq = torch.bincount(got, minlength=4).float() / got.numel()
    torch.testing.assert_close(freq, torch.tensor([2 / 3, 1 / 3, 0, 0], device=DEV), atol=0.02, rtol=0)


@pytest.mark.parametrize("n,target,controls", [(10, 0, ()), (10, 9, ()), (12, 5, (2,)), (12, 11, (0, 7)), (3, 1, (2,))])
def test_quantum_gate_kernel_matches_tensor_path(n, target, controls):
    """One-qubit and controlled gates of the quantum pack: streaming kernel against the matmul path."""
    from tensorplay_b200 import quantum as tq
    g = torch.Generator().manual_seed(n + target)
    s = torch.randn(3, 2 ** n, 2, generator=g)
    s = torch.view_as_complex(s / s.norm(dim=(1, 2), keepdim=True)).reshape([3] + [2] * n)
    u = tq.random_unitary(1, generator=g)
    ref = tq.apply_controlled(s, u, list(controls), target) if controls else tq.apply_gate(s, u, target)
    with torch.no_grad():
        sd, ud = s.to(DEV), u.to(DEV)
        out = tq.apply_controlled(sd, ud, list(controls), target) if controls else tq.apply_gate(sd, ud, target)
    torch.testing.assert_close(out.cpu(), ref, atol=1e-6, rtol=1e-5)
    from tensorplay_b200.quantum._native import apply_1q_native
    assert apply_1q_native(sd, ud, target, tuple(controls)) is not None   # the kernel is what ran


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("detach_reset", [False, True])
def test_fused_multi_step_lif_matches_cell_loop(dtype, detach_reset):
    """Fused LIF forward + BPTT against the per-step module under autograd (fp32 oracle on CPU)."""
    from tensorplay_b200 import snn
    T, B, N = 12, 3, 64
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(T, B, N, generator=g) * 1.5).to(dtype)
    gy = torch.randn(T, B, N, generator=g).to(dtype)
    # oracle: the time loop on CPU in fp32 from the same (rounded) inputs
    xr = x.float().clone().requires_grad_()
    cell = snn.LIFCell(tau=2.0, v_threshold=1.0, v_reset=0.0, alpha=2.0, detach_reset=detach_reset)
    v, out = None, []
    for t in range(T):
        s, v = cell(xr[t], v)
        out.append(s)
    ref = torch.stack(out)
    ref.backward(gy.float())
    xd = x.to(DEV).requires_grad_()
    lif = snn.LIF(tau=2.0, v_threshold=1.0, v_reset=0.0, alpha=2.0, detach_reset=detach_reset)
    sd = lif(xd)
    assert snn.multi_step_lif(xd.detach()) is not None            # the fused kernel is what ran
    sd.backward(gy.to(DEV))
    assert torch.equal(sd.float().cpu(), ref.detach())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(xd.grad.float().cpu(), xr.grad, atol=tol, rtol=tol)


def test_decode_qkv_prep_rotates_and_appends_in_one_launch():
    """q rotated out of the packed projection, k rotated into the key cache, v copied into the value cache, all at
    each sequence's own position; against the plain formulation of the same step."""
    import tensorplay_b200.ops as O
    torch.manual_seed(4)
    B, Hq, Hkv, D, S = 5, 8, 2, 128, 96
    qkv = torch.randn(B, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16)
    cos, sin = O.rope_tables(S, D, 500000.0, device="cuda")
    pos = torch.tensor([0, 7, 95, 33, 64], device="cuda", dtype=torch.int32)
    kc = torch.randn(B + 1, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn(B + 1, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
    kr, vr = kc.clone(), vc.clone()
    q = O.decode_qkv_prep(qkv, cos, sin, pos, Hq, Hkv, kc[:B], vc[:B])
    O.check_status()
    # reference: the CPU formulation of the same function
    qr = O.decode_qkv_prep(qkv.cpu(), cos.cpu(), sin.cpu(), pos.cpu(), Hq, Hkv, (kr := kr.cpu())[:B], (vr := vr.cpu())[:B])
    assert (q.cpu().float() - qr.float()).abs().max() < 0.04
    assert (kc.cpu().float() - kr.float()).abs().max() < 0.04          # untouched rows are bit-equal, new ones close
    assert torch.equal(vc.cpu(), vr)
    assert torch.equal(kc[B].cpu(), kr[B])                             # the row past the batch is untouched


def test_flash_fwd_writes_into_a_strided_output():
    """Decode attention with the query heads of a KV head as rows: the output lands directly in the [B, Hq * D]
    layout of the next projection, with and without split keys."""
    from tensorplay_b200.ops.attention import flash_fwd
    torch.manual_seed(5)
    B, Hkv, G, D, S = 3, 2, 4, 128, 1024
    q = torch.randn(B, Hkv * G, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device="cuda", dtype=torch.bfloat16)
    kv_len = torch.tensor(700, device="cuda", dtype=torch.int32)
    qv = q.view(B, Hkv, G, D).transpose(1, 2)
    for n_splits in (1, 4):
        ref, _ = flash_fwd(qv, k, v, False, D ** -0.5, kv_len=kv_len, n_splits=n_splits)
        ref = ref.transpose(1, 2).reshape(B, Hkv * G * D)
        out = torch.full((B, Hkv * G * D), float("nan"), device="cuda", dtype=torch.bfloat16)
        flash_fwd(qv, k, v, False, D ** -0.5, kv_len=kv_len, n_splits=n_splits, out=out.view(B, Hkv, G, D).transpose(1, 2))
        assert torch.equal(out, ref)
