"""AWQ scale search, pruning masks and the numeric comparison on CPU."""
import copy

import torch
from torch import nn

from tensorplay_b200 import quantization as Q


def _mlp(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(256, 256), nn.GELU(), nn.Linear(256, 128))


def test_awq_beats_plain_rounding_when_activations_have_outlier_channels():
    torch.manual_seed(0)
    lin = nn.Linear(256, 64, bias=False)
    x = torch.randn(512, 256)
    x[:, :8] *= 30.0                                   # a few dominant input channels
    scales, alpha, errs = Q.search_scales(lin.weight.data, x, bits=4, group_size=128)
    assert alpha > 0 and min(errs) < 0.7 * errs[0]     # errs[0]: alpha = 0 = plain group quantisation
    ref = x @ lin.weight.t()
    plain = Q.WeightOnlyLinear(copy.deepcopy(lin), 4, 128)(x)
    awq = Q.AWQLinear(lin, scales, 4, 128)(x)
    assert (awq - ref).pow(2).mean() < 0.7 * (plain - ref).pow(2).mean()


def test_awq_quantize_model_and_fold():
    m = _mlp()
    data = [torch.randn(64, 256) * torch.linspace(0.1, 5, 256) for _ in range(3)]
    ref = copy.deepcopy(m)
    chosen = Q.awq_quantize_(m, data, bits=4, group_size=128)
    assert set(chosen) == {"0", "2"} and isinstance(m[0], Q.AWQLinear)
    rep = Q.compare_models(ref, m, data[:1])
    assert rep["0"] > 15 and rep["2"] > 15             # dB
    # folding the division into a preceding norm leaves the function unchanged
    norm = nn.LayerNorm(256)
    lin = nn.Linear(256, 32)
    x = torch.randn(16, 256)
    s, _, _ = Q.search_scales(lin.weight.data, norm(x).detach(), 8, 128)
    q = Q.AWQLinear(lin, s, 8, 128)
    before = q(norm(x))
    q.fold_into(norm)
    torch.testing.assert_close(q(norm(x)), before, rtol=1e-4, atol=1e-4)


def test_masks_and_sparsifier_schedule():
    torch.manual_seed(1)
    w = torch.randn(64, 128)
    m = Q.magnitude_mask(w, 0.75)
    assert abs(m.float().mean().item() - 0.25) < 0.01 and w[m].abs().min() >= w[~m].abs().max()
    nm = Q.n_m_mask(w, 2, 4)
    assert bool((nm.reshape(-1, 4).sum(1) == 2).all())
    g = Q.global_magnitude_masks({"a": w, "b": w * 0.1}, 0.5)
    assert g["b"].float().mean() < g["a"].float().mean()
    model = _mlp(2)
    sp = Q.WeightSparsifier(model, pattern=(2, 4))
    sp.step()
    assert abs(sp.density() - 0.5) < 1e-6
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    for _ in range(3):                                  # updates cannot revive pruned weights
        opt.zero_grad()
        model(torch.randn(8, 256)).pow(2).mean().backward()
        opt.step()
    model(torch.randn(2, 256))
    assert bool((model[0].weight.data.reshape(-1, 4).ne(0).sum(1) <= 2).all())
    sp.squash()
    assert not sp.hooks
    s = [Q.cubic_sparsity(t, 100, 0.9) for t in (0, 50, 100)]
    assert s[0] == 0.0 and 0.7 < s[1] < 0.9 and abs(s[2] - 0.9) < 1e-12
    assert Q.sqnr(w, w + 0.01 * torch.randn_like(w)) > 35
