"""Fused multi-tensor SGD / Adagrad / RMSprop and the AMP kernels against torch's implementations."""
import pytest
import torch

import tensorplay_b200.optim as TO
from tensorplay_b200.amp import GradScaler
from tensorplay_b200.ops.optim import amp_unscale_, amp_update_scale_

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _params(dtype, seed=0):
    torch.manual_seed(seed)
    shapes = [(257, 33), (70000,), (5,), (128, 64)]   # more than one 65536-element chunk, odd sizes
    return [torch.randn(s, device=DEV).to(dtype).requires_grad_() for s in shapes]


CASES = [
    ("SGD", dict(lr=0.1)),
    ("SGD", dict(lr=0.05, momentum=0.9, weight_decay=0.01)),
    ("SGD", dict(lr=0.05, momentum=0.9, nesterov=True, dampening=0.0)),
    ("SGD", dict(lr=0.05, momentum=0.8, dampening=0.3, maximize=True)),
    ("Adagrad", dict(lr=0.1, lr_decay=0.01, weight_decay=0.01, eps=1e-8)),
    ("RMSprop", dict(lr=0.01, alpha=0.95)),
    ("RMSprop", dict(lr=0.01, momentum=0.9, centered=True, weight_decay=0.01)),
]


@pytest.mark.parametrize("name,kw", CASES)
def test_fused_optimizers_match_torch_fp32(name, kw):
    ours, ref = _params(torch.float32), _params(torch.float32)
    o1 = getattr(TO, name)(ours, **kw)
    o2 = getattr(torch.optim, name)(ref, **kw)
    for step in range(4):
        torch.manual_seed(100 + step)
        for a, b in zip(ours, ref):
            g = torch.randn_like(a)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    for a, b in zip(ours, ref):
        assert torch.allclose(a, b, rtol=2e-5, atol=2e-6), (name, kw, (a - b).abs().max().item())
    # state-dict layout is torch's: it loads into torch's optimizer
    o2.load_state_dict(o1.state_dict())


@pytest.mark.parametrize("name,kw", [CASES[1], CASES[4], CASES[6]])
def test_fused_optimizers_bf16_parameters_keep_fp32_master(name, kw):
    ours = _params(torch.bfloat16)
    ref = [p.detach().float().requires_grad_() for p in ours]
    o1 = getattr(TO, name)(ours, **kw)
    o2 = getattr(torch.optim, name)(ref, **kw)
    for step in range(6):
        torch.manual_seed(200 + step)
        for a, b in zip(ours, ref):
            g = torch.randn_like(b)
            a.grad, b.grad = g.to(torch.bfloat16), g.to(torch.bfloat16).float()
        o1.step()
        o2.step()
    for a, b in zip(ours, ref):
        assert torch.equal(a, b.to(torch.bfloat16)) or (a.float() - b).abs().max().item() < 2e-2
        assert torch.allclose(o1.state[a]["master"], b, rtol=2e-5, atol=2e-6)


def test_amp_unscale_and_scale_update():
    gs = [torch.randn(1000, device=DEV), torch.randn(70000, device=DEV), torch.randn(33, 7, device=DEV).to(torch.bfloat16)]
    want = [g.float() * 0.125 for g in gs]
    inv, found = torch.tensor([0.125], device=DEV), torch.zeros(1, device=DEV)
    amp_unscale_(gs, inv, found)
    assert float(found) == 0.0
    for g, w in zip(gs, want):
        assert torch.allclose(g.float(), w.to(g.dtype).float())
    gs[1][69999] = float("inf")
    amp_unscale_(gs, inv, found)
    assert float(found) == 1.0
    scale, tracker = torch.tensor([1024.0], device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    amp_update_scale_(scale, tracker, found, 2.0, 0.5, 3)
    assert float(scale) == 512.0 and int(tracker) == 0
    found.zero_()
    for k in range(3):
        amp_update_scale_(scale, tracker, found, 2.0, 0.5, 3)
    assert float(scale) == 1024.0 and int(tracker) == 0


def test_grad_scaler_with_fused_sgd_skips_non_finite_steps():
    torch.manual_seed(0)
    m = torch.nn.Linear(16, 8).to(DEV)
    ref = torch.nn.Linear(16, 8).to(DEV)
    ref.load_state_dict(m.state_dict())
    o1, o2 = TO.SGD(m.parameters(), lr=0.1, momentum=0.9), torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    s1 = GradScaler("cuda", init_scale=256.0, growth_interval=2)
    s2 = torch.amp.GradScaler("cuda", init_scale=256.0, growth_interval=2)
    x = torch.randn(4, 16, device=DEV)
    for step in range(5):
        for mod, opt, sc in ((m, o1, s1), (ref, o2, s2)):
            opt.zero_grad()
            loss = mod(x).pow(2).mean()
            sc.scale(loss).backward()
            if step == 2:
                mod.weight.grad[0, 0] = float("nan")   # this step must be skipped and the scale halved
            sc.step(opt)
            sc.update()
    assert float(s1.get_scale()) == float(s2.get_scale())
    assert torch.allclose(m.weight, ref.weight, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("kw", [dict(lr=1e-2), dict(lr=5e-3, weight_decay=0.05, d=1.5, eps=(1e-30, 1e-3)),
                                dict(lr=1e-2, maximize=True, beta2_decay=-0.6)])
def test_fused_adafactor_matches_torch(kw):
    """Factored (matrices) and plain (vectors) second moments, parameter-RMS step size and update clipping,
    all on the device, against torch.optim.Adafactor over several steps."""
    ours, ref = _params(torch.float32, seed=3), _params(torch.float32, seed=3)
    o1, o2 = TO.Adafactor(ours, **kw), torch.optim.Adafactor(ref, **kw)
    for step in range(5):
        torch.manual_seed(300 + step)
        for a, b in zip(ours, ref):
            g = torch.randn_like(a) * (0.1 + step)
            a.grad, b.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    for a, b in zip(ours, ref):
        assert torch.allclose(a, b, rtol=2e-4, atol=2e-5), (kw, a.shape, (a - b).abs().max().item())
        sa, sb = o1.state[a], o2.state[b]
        for key in ("row_var", "col_var", "variance"):
            if key in sb:
                assert torch.allclose(sa[key].view(-1), sb[key].view(-1), rtol=2e-4, atol=1e-7), key


def test_fused_adafactor_bf16_parameters():
    ours = _params(torch.bfloat16, seed=4)
    ref = [p.detach().float().requires_grad_() for p in ours]
    kw = dict(lr=1e-2, eps=(1e-30, 1e-3))   # the default eps1 is the dtype's epsilon, which differs between bf16 and fp32
    o1, o2 = TO.Adafactor(ours, **kw), torch.optim.Adafactor(ref, **kw)
    for step in range(4):
        torch.manual_seed(400 + step)
        for a, b in zip(ours, ref):
            g = torch.randn_like(b).to(torch.bfloat16)
            a.grad, b.grad = g, g.float()
        o1.step()
        o2.step()
    for a, b in zip(ours, ref):
        assert torch.allclose(o1.state[a]["master"], b, rtol=2e-4, atol=2e-5)
        assert (a.float() - b).abs().max().item() < 2e-2
