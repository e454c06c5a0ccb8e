"""BitNet b1.58: quantisers, packing, straight-through training, packed deployment; the integer product on the
tensor-core int8 GEMM against the fp32 product of the same integers."""
import pytest
import torch
from torch import nn

from tensorplay_b200.quantization import bitnet as B


def test_quantisers_and_packing():
    torch.manual_seed(0)
    w = torch.randn(6, 10)
    codes, scale = B.ternary_quantize(w)
    assert set(codes.unique().tolist()) <= {-1, 0, 1} and torch.isclose(scale, w.abs().mean())
    assert torch.equal(codes, torch.round(w / scale).clamp(-1, 1).to(torch.int8))
    packed = B.pack_ternary(codes)
    assert packed.shape == (6, 3) and packed.dtype == torch.uint8
    assert torch.equal(B.unpack_ternary(packed, 10), codes)
    x = torch.randn(4, 10)
    y = B.bitnet_linear(x, codes, scale=scale)
    xq = torch.round(x / (x.abs().amax(-1, keepdim=True) / 127)).clamp(-127, 127)
    want = (xq @ codes.float().t()) * (x.abs().amax(-1, keepdim=True) / 127) * scale
    assert torch.allclose(y, want, atol=1e-5)
    assert torch.allclose(B.bitnet_linear_packed(x, packed, scale, 10), y)


def test_straight_through_training_and_deployment():
    torch.manual_seed(1)
    lin = B.BitNetLinear(16, 5)
    x = torch.randn(7, 16, requires_grad=True)
    y = lin(x)
    g = torch.randn_like(y)
    y.backward(g)
    # gradients of the unquantised layer
    assert torch.allclose(x.grad, g @ lin.weight, atol=1e-5) and torch.allclose(lin.weight.grad, g.t() @ x, atol=1e-5)
    assert torch.allclose(lin.bias.grad, g.sum(0), atol=1e-6)
    packed = lin.pack()
    assert packed.shape == (5, 16) and packed.nbytes() == 5 * 4 + 4
    assert torch.allclose(packed.linear(x.detach(), lin.bias.detach()), y.detach(), atol=1e-5)
    assert (packed.dequantize() - lin.weight.detach()).abs().mean() < lin.weight.detach().abs().mean()
    # a model converted in place trains: the loss of a small regression goes down
    net = nn.Sequential(nn.Linear(8, 32), nn.ReLU(), nn.Linear(32, 1))
    B.quantize_(net, B.BitNetTrainingConfig())
    assert isinstance(net[0].weight, B.BitNetTrainingLinearWeight)
    opt = torch.optim.Adam(net.parameters(), lr=1e-2)
    data, target = torch.randn(256, 8), None
    target = data[:, :1] * 2 - data[:, 1:2]
    losses = []
    for _ in range(150):
        loss = (net(data) - target).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.5 * losses[0]
    codes, _ = B.ternary_quantize(net[0].weight.detach())
    assert set(codes.unique().tolist()) <= {-1, 0, 1}
    from_lin = B.BitNetLinear.from_linear(nn.Linear(4, 3))
    assert from_lin(torch.randn(2, 4)).shape == (2, 3)


@pytest.mark.gpu
def test_integer_product_on_the_int8_tensor_core_gemm():
    torch.manual_seed(2)
    lin = B.BitNetLinear(512, 384, device="cuda", dtype=torch.bfloat16)
    x = torch.randn(3, 40, 512, device="cuda", dtype=torch.bfloat16)
    y = lin(x)
    codes, scale = B.ternary_quantize(lin.weight.detach())
    xq, sx = B._act_quantize(x)
    want = (xq.float() @ codes.float().t()) * sx * scale + lin.bias.float()
    assert y.shape == (3, 40, 384) and y.dtype == torch.bfloat16
    assert (y.float() - want).abs().max() <= 2 ** -7 * want.abs().max() + 1e-3        # bf16 output rounding only
    packed = lin.pack()
    assert torch.equal(packed.linear(x, lin.bias.detach()), y)
