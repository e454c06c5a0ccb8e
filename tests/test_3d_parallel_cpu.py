"""Tensor x pipeline x data parallel composed on eight gloo ranks (TP2 x PP2 x FSDP2), against the dense
single-process model: losses of two optimizer steps and the updated weights must agree.

rank = pp * 4 + dp * 2 + tp. Each pipeline stage is one tensor-parallel Llama block with
sequence-parallel rows, its parameters sharded over the data-parallel pair by ``fully_shard``;
micro-batches run under the 1F1B schedule.
"""
import torch
from torch import nn

from tests.distutil import run_ranks

TP, DP, PP = 2, 2, 2
B, T, MB = 4, 8, 2           # per data-parallel rank: 4 sequences in 2 micro-batches
LR = 0.05


def _cfg():
    from tensorplay_b200.models.llama import LlamaConfig
    return LlamaConfig.tiny(hidden_size=32, num_heads=4, num_kv_heads=2, head_dim=8, ffn_size=48, vocab_size=64,
                            num_layers=PP, max_seq_len=T)


def _dense(cfg):
    from tensorplay_b200.models.llama import LlamaBlock
    g = torch.Generator().manual_seed(11)
    blocks = [LlamaBlock(cfg, i) for i in range(PP)]
    for b in blocks:
        b.reset_parameters(g)
        with torch.no_grad():  # non-trivial norm weights so that their gradients matter
            b.attn_norm.add_(0.1 * torch.randn(b.attn_norm.shape, generator=g))
            b.ffn_norm.add_(0.1 * torch.randn(b.ffn_norm.shape, generator=g))
    return blocks


def _data(cfg):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(DP, B, T, cfg.hidden_size, generator=g)
    y = torch.randn(DP, B, T, cfg.hidden_size, generator=g)
    return x, y


def _tp_slices(cfg, ld, r):
    """This tensor-parallel rank's slices of a dense block's weights (heads and FFN columns)."""
    D, Hq, Hkv, F = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.ffn_size
    hq, hkv, ff = Hq // TP, Hkv // TP, F // TP
    q = ld.wqkv[: Hq * D].view(Hq, D, -1)[r * hq: (r + 1) * hq].reshape(hq * D, -1)
    k = ld.wqkv[Hq * D: (Hq + Hkv) * D].view(Hkv, D, -1)[r * hkv: (r + 1) * hkv].reshape(hkv * D, -1)
    v = ld.wqkv[(Hq + Hkv) * D:].view(Hkv, D, -1)[r * hkv: (r + 1) * hkv].reshape(hkv * D, -1)
    g, u = ld.w_gate_up[:F], ld.w_gate_up[F:]
    return {"attn_norm": ld.attn_norm, "ffn_norm": ld.ffn_norm, "wqkv": torch.cat((q, k, v), 0),
            "wo": ld.wo[:, r * hq * D: (r + 1) * hq * D],
            "w_gate_up": torch.cat((g[r * ff: (r + 1) * ff], u[r * ff: (r + 1) * ff]), 0),
            "w_down": ld.w_down[:, r * ff: (r + 1) * ff]}


def _dense_reference():
    """Two SGD steps of the dense two-block model on the whole batch: losses and final weights."""
    from tensorplay_b200 import ops
    cfg = _cfg()
    blocks = _dense(cfg)
    x, y = _data(cfg)
    cos, sin = ops.rope_tables(T, cfg.head_dim, cfg.rope_theta)
    params = [p for b in blocks for p in b.parameters()]
    opt = torch.optim.SGD(params, lr=LR)
    losses = []
    for _ in range(2):
        opt.zero_grad()
        h = x.reshape(DP * B, T, -1)
        for b in blocks:
            h = b(h, cos, sin)
        loss = ((h - y.reshape(DP * B, T, -1)) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, blocks


class _Stage(nn.Module):
    """One tensor-parallel block; the first stage cuts its rows out of the replicated input."""

    def __init__(self, block, first, cos, sin):
        super().__init__()
        self.block, self.first = block, first
        self.cos, self.sin = cos, sin

    def forward(self, x):
        tp = self.block.tp
        b = B // MB
        if self.first:
            rows = x.reshape(b * T, -1)
            n = rows.shape[0] // tp.world
            x = rows[tp.rank * n: (tp.rank + 1) * n]
        return self.block(x, b, T, self.cos, self.sin)


def _worker(rank, world):
    import torch.distributed as dist
    from tensorplay_b200 import ops
    from tensorplay_b200.distributed.fsdp import fully_shard
    from tensorplay_b200.distributed.pipelining import PipelineStage, Schedule1F1B
    from tensorplay_b200.models.llama_tp import LlamaTPBlock
    from tensorplay_b200.parallel.tp import TPContext
    pp, dp, tp = rank // 4, (rank // 2) % 2, rank % 2
    tp_group = dp_group = pp_group = None
    for p in range(PP):                      # every rank creates every group, in the same order
        for d in range(DP):
            g = dist.new_group([p * 4 + d * 2 + t for t in range(TP)])
            if (p, d) == (pp, dp):
                tp_group = g
    for p in range(PP):
        for t in range(TP):
            g = dist.new_group([p * 4 + d * 2 + t for d in range(DP)])
            if (p, t) == (pp, tp):
                dp_group = g
    for d in range(DP):
        for t in range(TP):
            g = dist.new_group([p * 4 + d * 2 + t for p in range(PP)])
            if (d, t) == (dp, tp):
                pp_group = g

    cfg = _cfg()
    dense = _dense(cfg)
    ctx = TPContext(group=tp_group)
    assert (ctx.world, ctx.rank) == (TP, tp)
    block = LlamaTPBlock(cfg, ctx, pp)
    with torch.no_grad():
        for name, w in _tp_slices(cfg, dense[pp], tp).items():
            getattr(block, name).copy_(w)
    cos, sin = ops.rope_tables(T, cfg.head_dim, cfg.rope_theta)
    stage_mod = _Stage(block, pp == 0, cos, sin)
    fully_shard(stage_mod, process_group=dp_group)
    opt = torch.optim.SGD(stage_mod.parameters(), lr=LR)

    x, y = _data(cfg)
    n_loc = (B // MB) * T // TP

    def loss_fn(out, target):
        # this rank's rows of the micro-batch; the two tensor-parallel ranks' parts add up to the MSE
        t = target.reshape(-1, target.shape[-1])[tp * n_loc: (tp + 1) * n_loc]
        return ((out - t) ** 2).sum() / target.numel()

    stage = PipelineStage(stage_mod, pp, PP, group=pp_group)
    sched = Schedule1F1B(stage, MB, loss_fn=loss_fn)
    step_losses = []
    for _ in range(2):
        opt.zero_grad()
        losses = []
        if pp == 0:
            sched.step(x[dp])
        else:
            sched.step(target=y[dp], losses=losses)
        # sequence parallelism: a replicated weight saw only this rank's rows
        for n, p in stage_mod.named_parameters():
            if n.endswith("norm"):
                dist.all_reduce(p.grad, group=tp_group)
        opt.step()
        if pp == PP - 1:
            l = torch.stack(losses).mean()       # this rank's share of the data-parallel rank's MSE
            dist.all_reduce(l, group=tp_group)   # + the other rows
            dist.all_reduce(l, group=dp_group)   # mean over the data-parallel ranks
            step_losses.append(l.item() / DP)
    stage_mod.unshard()
    final = {n: getattr(block, n).detach().clone().numpy() for n in
             ("attn_norm", "ffn_norm", "wqkv", "wo", "w_gate_up", "w_down")}
    dist.barrier()
    return pp, tp, step_losses, final


def test_tp2_pp2_fsdp2_matches_dense_model():
    ref_losses, ref_blocks = _dense_reference()
    assert ref_losses[1] < ref_losses[0]
    out = run_ranks(_worker, TP * DP * PP, timeout=300.0)
    cfg = _cfg()
    for pp, tp, losses, final in out:
        if pp == PP - 1:
            for a, b in zip(losses, ref_losses):
                assert abs(a - b) < 1e-5 * max(1.0, abs(b)), (losses, ref_losses)
        want = _tp_slices(cfg, ref_blocks[pp], tp)
        for name, w in final.items():
            torch.testing.assert_close(torch.from_numpy(w), want[name].detach(), rtol=1e-4, atol=1e-5)
