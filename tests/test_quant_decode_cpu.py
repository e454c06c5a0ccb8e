"""CPU oracles of the quantised / decode ops and the modules built on them."""
import torch

import tensorplay_b200.ops as O
from tensorplay_b200 import quantization as Q
from tensorplay_b200.nn.cache import PagedCache, StaticCache


def test_weight_quantisers_round_trip():
    w = torch.randn(64, 256)
    q, s = O.quantize_weight_int8(w, 64)
    assert (O.dequantize_weight(q, s, None, 8, 64).float() - w).abs().max() < 0.05
    p, s4, z4 = O.quantize_weight_int4(w, 64)
    assert p.shape == (64, 128) and (O.dequantize_weight(p, s4, z4, 4, 64).float() - w).abs().max() < 0.5


def test_quantize_module_swap():
    m = torch.nn.Sequential(torch.nn.Linear(128, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32)).bfloat16()
    x = torch.randn(4, 128).bfloat16()
    ref = m(x).float()
    for mode, tol in [("int8_weight_only", 0.1), ("int4_weight_only", 0.6), ("int8_dynamic", 0.15),
                      ("float8_weight_only", 0.2)]:
        import copy
        qm = Q.quantize_(copy.deepcopy(m), mode, group_size=64 if "int4" in mode else 0)
        assert not any(isinstance(c, torch.nn.Linear) for c in qm.modules())
        assert (qm(x).float() - ref).abs().max() < tol, mode


def test_sample_reference_support_rules():
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0]]).log_softmax(-1)
    # u = 0 picks the first supported index, u -> 1 the last supported one
    assert O.sample(logits, 1.0, 2, 1.0, uniform=torch.tensor([0.999])).item() == 1
    assert O.sample(logits, 1.0, 0, 0.5, uniform=torch.tensor([0.999])).item() == 0
    assert O.sample(logits, 1.0, 0, 1.0, uniform=torch.tensor([0.0])).item() == 0


def test_caches_agree():
    k = torch.randn(2, 2, 5, 8); v = torch.randn(2, 2, 5, 8)
    sc, pc = StaticCache(16), PagedCache(block_size=4)
    for c in (sc, pc):
        c.update(k[:, :, :3], v[:, :, :3])
        kk, vv = c.update(k[:, :, 3:], v[:, :, 3:])
        torch.testing.assert_close(kk, k)
        torch.testing.assert_close(vv, v)
