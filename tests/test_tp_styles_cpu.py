"""``parallelize_module`` with column / row styles on the module-level decoder, two gloo ranks:
forward, loss and gradients equal the dense model's (weights gathered back for the comparison)."""
import copy

import torch

from tests.distutil import run_ranks


def _worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200 import nn
    from tensorplay_b200.distributed.tensor.parallel import ColwiseParallel, RowwiseParallel, parallelize_module
    torch.manual_seed(0)
    dense = nn.DecoderLM(64, 32, 2, 4, 2, intermediate_size=48)
    tp = copy.deepcopy(dense)
    rep_in = ColwiseParallel(input_sharded=False)       # replicated activations in, heads / columns out
    red_out = RowwiseParallel(output_sharded=False)     # partial sums all-reduced back to replicated
    plan = {"layers.*.mixer.q_proj": rep_in, "layers.*.mixer.k_proj": rep_in, "layers.*.mixer.v_proj": rep_in,
            "layers.*.mixer.o_proj": red_out, "layers.*.mlp.gate_proj": rep_in, "layers.*.mlp.up_proj": rep_in,
            "layers.*.mlp.down_proj": red_out}
    parallelize_module(tp, None, plan)
    assert tp.layers[0].mixer.num_heads == 2 and tp.layers[0].mixer.num_kv_heads == 1
    assert tp.layers[0].mlp.gate_proj.weight.shape == (24, 32) and tp.layers[0].mlp.down_proj.weight.shape == (32, 24)
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(0, 64, (2, 9), generator=g)
    torch.testing.assert_close(tp(tok), dense(tok), rtol=1e-4, atol=1e-5)
    l_tp, l_d = tp(tok[:, :-1], tok[:, 1:]), dense(tok[:, :-1], tok[:, 1:])
    torch.testing.assert_close(l_tp, l_d, rtol=1e-5, atol=1e-6)
    l_tp.backward()
    l_d.backward()
    # a column shard's gradient is the matching slice of the dense gradient; replicated parameters
    # (embedding, norms, head) see the full gradient on every rank
    n = 24
    torch.testing.assert_close(tp.layers[1].mlp.up_proj.weight.grad,
                               dense.layers[1].mlp.up_proj.weight.grad[rank * n: (rank + 1) * n], rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(tp.layers[0].mlp.down_proj.weight.grad,
                               dense.layers[0].mlp.down_proj.weight.grad[:, rank * n: (rank + 1) * n], rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(tp.layers[0].mixer.o_proj.weight.grad,
                               dense.layers[0].mixer.o_proj.weight.grad[:, rank * 16: (rank + 1) * 16], rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(tp.embed.weight.grad, dense.embed.weight.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(tp.norm.weight.grad, dense.norm.weight.grad, rtol=1e-4, atol=1e-6)
    # cached generation through the sharded model equals the dense one
    a = nn.generate(tp, tok[:, :4], max_new_tokens=4)
    b = nn.generate(dense, tok[:, :4], max_new_tokens=4)
    assert torch.equal(a, b)
    dist.barrier()
    return True


def test_parallelize_module_on_decoder_lm():
    assert all(run_ranks(_worker, 2))


def _prepare_worker(rank, world):
    import torch.distributed as dist
    from torch import nn as tnn
    from tensorplay_b200.distributed.tensor.parallel import (ColwiseParallel, PrepareModuleInput, PrepareModuleInputOutput,
                                                             PrepareModuleOutput, RowwiseParallel, input_reshard,
                                                             parallelize_module)
    torch.manual_seed(0)

    class MLP(tnn.Module):
        def __init__(self):
            super().__init__()
            self.up, self.down = tnn.Linear(16, 32, bias=False), tnn.Linear(32, 16, bias=False)

        def forward(self, x):
            return self.down(torch.tanh(self.up(x)))
    dense = MLP()
    tp = copy.deepcopy(dense)
    # sequence-sharded rows in and out; replicated inside the block
    parallelize_module(tp, None, {
        "": PrepareModuleInputOutput(input_layouts="shard", desired_input_layouts="replicate",
                                     output_layouts="replicate", desired_output_layouts="shard"),
        "up": ColwiseParallel(input_sharded=False), "down": RowwiseParallel(output_sharded=False)})
    x = torch.randn(8, 16, generator=torch.Generator().manual_seed(1))
    xl = x[rank * 4: (rank + 1) * 4].clone().requires_grad_()
    xd = x.clone().requires_grad_()
    y = tp(xl)
    yd = dense(xd)
    torch.testing.assert_close(y, yd[rank * 4: (rank + 1) * 4], rtol=1e-5, atol=1e-6)
    # the loss is the sum over all rows: each rank contributes its rows
    y.pow(2).sum().backward()
    yd.pow(2).sum().backward()
    torch.testing.assert_close(xl.grad, xd.grad[rank * 4: (rank + 1) * 4], rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(tp.up.weight.grad, dense.up.weight.grad[rank * 16: (rank + 1) * 16], rtol=1e-4, atol=1e-6)
    # placement objects are accepted as layouts; the single-direction styles compose the same way
    from torch.distributed.tensor import Replicate, Shard
    m2 = copy.deepcopy(dense)
    parallelize_module(m2, None, {"": PrepareModuleInput(input_layouts=Shard(0), desired_input_layouts=Replicate())})
    parallelize_module(m2, None, {"": PrepareModuleOutput(output_layouts=Replicate(), desired_output_layouts=Shard(0))})
    torch.testing.assert_close(m2(x[rank * 4: (rank + 1) * 4]), yd[rank * 4: (rank + 1) * 4].detach(), rtol=1e-5, atol=1e-6)
    # input_reshard: same gradients, the saved input is a slice
    m3, m4 = copy.deepcopy(dense), copy.deepcopy(dense)
    input_reshard(m3.up, None, 0, group=dist.group.WORLD)
    a = x.clone().requires_grad_()
    b = x.clone().requires_grad_()
    m3(a).pow(2).sum().backward()
    m4(b).pow(2).sum().backward()
    torch.testing.assert_close(a.grad, b.grad)
    torch.testing.assert_close(m3.up.weight.grad, m4.up.weight.grad)
    dist.barrier()
    return True


def test_prepare_module_styles_and_input_reshard():
    assert all(run_ranks(_prepare_worker, 2))
