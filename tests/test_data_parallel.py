"""Single-process data parallelism: the pieces' gradients add up in the one set of parameters."""
import pytest
import torch
from torch import nn

from tensorplay_b200.nn.parallel import DataParallel, data_parallel, gather, scatter


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 8), nn.BatchNorm1d(8), nn.Tanh(), nn.Linear(8, 3))


def test_matches_the_full_batch_on_cpu_devices():
    net, ref = _net().eval(), _net().eval()            # eval: batch-norm statistics are not per piece
    dp = DataParallel(net, device_ids=["cpu", "cpu", "cpu"])
    x = torch.randn(10, 6)
    y = dp(x)
    yr = ref(x)
    assert torch.allclose(y, yr, atol=1e-6)
    y.square().sum().backward()
    yr.square().sum().backward()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-5)
    # containers, keyword arguments, a batch smaller than the device count
    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(6, 2)

        def forward(self, x, scale=None):
            out = self.l(x)
            return {"out": out * scale if scale is not None else out, "norm": out.norm()}
    m = Two()
    res = data_parallel(m, (x,), ["cpu", "cpu"], module_kwargs={"scale": torch.arange(10.0).view(10, 1)})
    assert res["out"].shape == (10, 2) and res["norm"].shape == (2,)
    assert torch.allclose(res["out"], m.l(x) * torch.arange(10.0).view(10, 1), atol=1e-6)
    assert DataParallel(m, ["cpu"] * 4)(x[:2])["out"].shape == (2, 2)
    assert [t.shape[0] for t in scatter(torch.zeros(7, 2), ["cpu", "cpu", "cpu"])] == [3, 3, 1]
    assert gather([torch.ones(2, 2), torch.zeros(1, 2)], "cpu").shape == (3, 2)
    assert DataParallel(m, device_ids=[])(x)["out"].shape == (10, 2)


@pytest.mark.gpu
def test_two_gpus_accumulate_into_one_parameter_set():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    net, ref = _net().eval().cuda(0), _net().eval().cuda(0)
    dp = DataParallel(net, device_ids=[0, 1])
    x = torch.randn(16, 6, device="cuda:0")
    y, yr = dp(x), ref(x)
    assert y.device == torch.device("cuda:0") and torch.allclose(y, yr, atol=1e-5)
    y.square().sum().backward()
    yr.square().sum().backward()
    for p, q in zip(net.parameters(), ref.parameters()):
        assert torch.allclose(p.grad, q.grad, atol=1e-4)
    with pytest.raises(RuntimeError):
        DataParallel(_net().cuda(1), device_ids=[0, 1])
