"""snn pack on CPU: neuron dynamics against hand-rolled recurrences, surrogates, encoders, monitor."""
import math

import torch
from torch import nn

from tensorplay_b200 import snn


def test_lif_node_single_and_multi_step_agree_and_keep_state():
    torch.manual_seed(0)
    x = torch.rand(10, 3, 8) * 1.5
    single = snn.LIFNode(threshold=1.0, decay=0.6)
    multi = snn.LIFNode(threshold=1.0, decay=0.6, step_mode="m", return_v_seq=True)
    s1 = torch.stack([single(x[t]) for t in range(10)])
    s2, v_seq = multi(x)
    assert torch.equal(s1, s2)
    torch.testing.assert_close(single.v, multi.v)
    torch.testing.assert_close(v_seq[-1], multi.v)
    # hand-rolled recurrence (hard reset to 0)
    v, ref = torch.zeros(3, 8), []
    for t in range(10):
        h = 0.6 * v + x[t]
        s = (h >= 1.0).float()
        v = h * (1 - s)
        ref.append(s)
    assert torch.equal(s1, torch.stack(ref))
    # state carries over a second call; reset() clears it
    again = multi(x)[0]
    multi.reset()
    fresh = multi(x)[0]
    assert torch.equal(fresh, s2) and not torch.equal(again, s2)


def test_soft_reset_if_and_parametric_nodes():
    x = torch.full((6, 1, 4), 0.7)
    soft = snn.IFNode(threshold=1.0, v_reset=None, step_mode="m")
    s = soft(x)
    # integrate 0.7 per step, subtract 1 at each spike: spikes at steps 1, 2, 4, 5 (0-based)
    assert s[:, 0, 0].tolist() == [0.0, 1.0, 1.0, 0.0, 1.0, 1.0]
    plif = snn.ParametricLIFNode(init_decay=0.5, step_mode="m", surrogate=snn.SigmoidSurrogate())
    torch.testing.assert_close(torch.sigmoid(plif.w.detach()), torch.tensor(0.5))
    out = plif(torch.rand(5, 2, 4, generator=torch.Generator().manual_seed(1)) * 2)
    out.sum().backward()
    assert plif.w.grad is not None and plif.w.grad.abs() > 0
    th = snn.LIFNode(learnable_threshold=True, step_mode="m", surrogate=snn.ATanSurrogate())
    th(torch.rand(5, 2, 4) * 2).sum().backward()
    assert th.threshold.grad is not None


def test_alif_threshold_adapts():
    x = torch.full((20, 1, 1), 1.2)
    lif = snn.LIFNode(decay=0.0, step_mode="m")(x)
    alif = snn.ALIFNode(decay=0.0, rho=0.9, beta=0.5, step_mode="m")(x)
    assert lif.sum() == 20 and alif.sum() < 20     # the rising threshold suppresses spikes


def test_surrogates_are_bumps_around_the_threshold():
    u = torch.linspace(-3, 3, 601, dtype=torch.float64)
    assert len(set(snn.SURROGATES.values())) == 15
    for name, cls in snn.SURROGATES.items():
        sg = cls()
        g = sg.grad(u)
        assert g.shape == u.shape and torch.isfinite(g).all(), name
        if name not in ("LeakyKRELUSurrogate", "S2NNSurrogate", "FourierSeriesSurrogate"):
            assert g[300] >= g[0] and g[300] >= g[-1], name        # peak at the threshold
        x = torch.tensor([-0.2, 0.3], requires_grad=True)
        y = sg(x)
        assert y.tolist() == [0.0, 1.0]
        y.sum().backward()
        torch.testing.assert_close(x.grad, sg.grad(x.detach()))
    # sigmoid / arctan / erf surrogates are derivatives of unit steps: they integrate to 1
    for cls in (snn.SigmoidSurrogate, snn.ErfSurrogate, snn.PiecewiseLinearSurrogate, snn.PiecewiseExpSurrogate):
        wide = torch.linspace(-40, 40, 160001, dtype=torch.float64)
        assert abs(torch.trapezoid(cls().grad(wide), wide).item() - 1.0) < 1e-3, cls.__name__
    assert abs(snn.ATanSurrogate(2.0).grad(torch.zeros(1)).item() - 1.0) < 1e-6


def test_encoders():
    g = torch.Generator().manual_seed(0)
    x = torch.tensor([0.0, 0.25, 1.0])
    r = snn.rate_encode(x, 4000, generator=g)
    torch.testing.assert_close(r.mean(0), x, atol=0.03, rtol=0)
    lat = snn.temporal_encode(x, 5)
    assert lat.sum(0).tolist() == [1.0, 1.0, 1.0] and lat[:, 2].argmax() == 0 and lat[:, 0].argmax() == 4
    assert snn.LatencyEncoder(5, "log")(x).sum(0).tolist() == [1.0, 1.0, 1.0]
    wp = snn.WeightedPhaseEncoder(8)
    v = torch.tensor([0.0, 0.3125, 0.7])
    torch.testing.assert_close(wp.decode(wp(v)), v, atol=2 ** -8, rtol=0)
    per = snn.PeriodicEncoder(torch.tensor([[1.0], [0.0], [0.0]]))
    assert per(7)[:, 0].tolist() == [1.0, 0.0, 0.0, 1.0, 0.0, 0.0, 1.0]
    gt = snn.GaussianTuningCurveEncoder(0.0, 1.0, m=6, steps=8)
    sp = gt(torch.tensor([0.5]))
    assert sp.shape == (8, 1, 6) and sp.sum() == 6      # every population neuron fires once


def test_sequence_layers_monitor_and_rate_loss():
    torch.manual_seed(0)
    net = nn.Sequential(snn.SpikingConv2d(1, 4, 3, padding=1), snn.SpikingBatchNorm2d(4),
                        snn.LIFNode(step_mode="m", surrogate=snn.ATanSurrogate()),
                        snn.SeqToANNContainer(nn.Flatten(), snn.SpikeLinear(4 * 6 * 6, 10)),
                        snn.LIFNode(step_mode="m", surrogate=snn.ATanSurrogate()))
    x = snn.rate_encode(torch.rand(2, 1, 6, 6), 5)
    with snn.SpikeMonitor(net) as mon:
        out = net(x)
        rates = mon.rates()
    assert out.shape == (5, 2, 10) and set(rates) == {"2", "4"} and all(0 <= r <= 1 for r in rates.values())
    loss = snn.spike_rate_loss(out, 0.2)
    loss.backward()
    assert net[0][0].weight.grad is not None and torch.isfinite(net[0][0].weight.grad).all()
    assert abs(snn.spike_rate(out).mean().item() - out.mean().item()) < 1e-6


def test_tau_layer_matches_decay_node():
    # v + (x - v) / tau == decay v + x / tau with decay = 1 - 1 / tau
    x = torch.rand(7, 2, 8, generator=torch.Generator().manual_seed(2)) * 3
    a = snn.LIF(tau=2.0)(x)
    b = snn.LIFNode(decay=0.5, step_mode="m")(x / 2.0)
    assert torch.equal(a, b)
