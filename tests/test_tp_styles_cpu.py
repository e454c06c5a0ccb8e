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
