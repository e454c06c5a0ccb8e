"""quantize_ workflows: each configuration swaps the linear layers, outputs stay close to the float model, int8 mixed
precision trains."""
import pytest
import torch
from torch import nn

from tensorplay_b200.quantization import workflows as W


def _mlp(d=64, h=128):
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(d, h), nn.GELU(), nn.Linear(h, d))


@pytest.mark.parametrize("config,layer,tol", [
    (W.Int8WeightOnlyQuantizedTrainingConfig(), W.Int8WeightOnlyQuantizedLinear, 0.02),
    (W.Int4WeightOnlyConfig(group_size=32), W.WeightOnlyInt4Linear, 0.12),
    (W.Float8WeightOnlyConfig(), W.Float8WeightOnlyInferenceLinear, 0.06),
    (W.float8_dynamic_activation_float8_weight, W.Float8DynamicActivationInferenceLinear, 0.09),
    (W.Int2WeightOnlyConfig(group_size=16), W.WeightOnlyInt2Linear, 0.45),
    (W.BinaryWeightOnlyConfig(), W.BinaryWeightOnlyLinear, 0.85),
])
def test_inference_configs_stay_close_to_the_float_model(config, layer, tol):
    ref, net = _mlp(), _mlp()
    W.quantize_(net, config)
    assert isinstance(net[0], layer) and isinstance(net[2], layer)
    x = torch.randn(5, 64)
    y, yr = net(x), ref(x)
    assert (y - yr).norm() / yr.norm() < tol
    # a filter leaves the rest alone
    net2 = _mlp()
    W.quantize_(net2, config, filter_fn=lambda m, name: name == "2")
    assert type(net2[0]) is nn.Linear and isinstance(net2[2], layer)


def test_int8_mixed_precision_training_follows_the_float_run():
    ref, net = _mlp(), _mlp()
    W.quantize_(net, W.int8_mixed_precision_training(output=True, grad_input=True, grad_weight=True))
    assert isinstance(net[0], W.Int8MixedPrecisionTrainingLinear) and net[0].weight is not None
    x = torch.randn(32, 64)
    t = torch.randn(32, 64)
    y, yr = net(x), ref(x)
    assert (y - yr).norm() / yr.norm() < 0.03
    (y - t).pow(2).mean().backward()
    (yr - t).pow(2).mean().backward()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert (p.grad - q.grad).norm() / q.grad.norm() < 0.06
    # the same SGD run on both models: the int8 run tracks the float run
    def run(model):
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        curve = []
        for _ in range(60):
            loss = (model(x) - t).pow(2).mean()
            opt.zero_grad()
            loss.backward()
            opt.step()
            curve.append(float(loss.detach()))
        return curve
    cq, cf = run(net), run(ref)
    assert cq[-1] < cq[0] and abs(cq[-1] - cf[-1]) < 0.02 * cf[-1]
    with pytest.raises(TypeError):
        W.quantize_(_mlp(), object())


@pytest.mark.gpu
def test_int8_mixed_precision_on_the_tensor_core_gemm():
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 256)).cuda().bfloat16()
    net = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 256)).cuda().bfloat16()
    net.load_state_dict(ref.state_dict())
    W.quantize_(net, W.Int8MixedPrecisionTrainingConfig())
    x = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16)
    y, yr = net(x), ref(x)
    assert (y.float() - yr.float()).norm() / yr.float().norm() < 0.04
    y.float().pow(2).mean().backward()
    yr.float().pow(2).mean().backward()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert (p.grad.float() - q.grad.float()).norm() / q.grad.float().norm() < 0.08
    w4 = nn.Sequential(nn.Linear(256, 512)).cuda().bfloat16()
    r4 = w4[0](x[:4])
    W.quantize_(w4, W.Int4WeightOnlyConfig(group_size=128))
    assert (w4(x[:4]).float() - r4.float()).norm() / r4.float().norm() < 0.15     # decode-sized: the GEMV kernel


def test_two_bit_packing_round_trip():
    codes = torch.randint(0, 4, (5, 13))
    assert torch.equal(W.unpack_int2(W.pack_int2(codes), 13), codes.to(torch.uint8))
    w = torch.randn(6, 32)
    q, s, z = W.quantize_int2_weight_only(w, 16)
    lin = nn.Linear(32, 6, bias=False)
    with torch.no_grad():
        lin.weight.copy_(w)
    m = W.WeightOnlyInt2Linear(lin, 16)
    assert q.shape == (6, 8) and (m.dequantize() - w).abs().max() <= s.max() / 2 + 1e-6     # half a step at most
    b = W.BinaryWeightOnlyLinear(lin)
    assert torch.equal(torch.sign(b.dequantize()), torch.where(w >= 0, 1.0, -1.0)) and b.qweight.shape == (6, 4)

