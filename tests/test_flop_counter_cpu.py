"""The FLOP counter books the native kernels' work (reported by the op wrappers) next to ATen operators."""
import torch

from tensorplay_b200 import _native
from tensorplay_b200.utils.flop_counter import FlopCounterMode


def test_native_flops_are_attributed_to_the_running_module():
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = torch.nn.Linear(8, 4, bias=False)

        def forward(self, x):
            # what an op wrapper does after its launch
            if _native.flop_sinks:
                _native.add_flops("tpb.gemm", 1000)
            return self.lin(x)

    net = torch.nn.Sequential(Block(), torch.nn.ReLU())
    with FlopCounterMode(net, display=False) as fc:
        net(torch.randn(2, 8))
    aten = 2 * 2 * 8 * 4
    assert fc.get_total_flops() == 1000 + aten
    counts = fc.get_flop_counts()
    assert counts["Global"]["tpb.gemm"] == 1000
    block = [k for k in counts if k.endswith("0")][0]
    assert counts[block]["tpb.gemm"] == 1000
    assert "tpb.gemm" in fc.get_table()
    assert not _native.flop_sinks                       # deregistered on exit
    _native.add_flops("tpb.gemm", 5)                    # no counter active: dropped
    assert fc.get_total_flops() == 1000 + aten


def test_cpu_fallback_ops_are_counted_by_the_dispatcher():
    import tensorplay_b200.ops as O
    a, b = torch.randn(16, 32), torch.randn(24, 32)
    with FlopCounterMode(display=False) as fc:
        O.gemm(a, b)
    assert fc.get_total_flops() == 2 * 16 * 24 * 32
