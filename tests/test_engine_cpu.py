"""The sharded engine against plain autograd + torch AdamW on CPU (single rank)."""
import copy

import torch

from tensorplay_b200.models.llama import Llama, LlamaConfig
from tensorplay_b200.parallel import AdamWConfig, FSDPEngine


def _run_ref(model, tokens, targets, steps, cfg):
    opt = torch.optim.AdamW(model.parameters(), lr=cfg.lr, betas=cfg.betas, eps=cfg.eps,
                            weight_decay=cfg.weight_decay)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(tokens, targets)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


def test_engine_matches_autograd_single_rank():
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(num_layers=3)
    model = Llama(cfg)
    model.reset_parameters(0)
    ref = copy.deepcopy(model)
    tokens = torch.randint(0, cfg.vocab_size, (2, 24))
    targets = torch.randint(0, cfg.vocab_size, (2, 24))
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref_losses = _run_ref(ref, tokens, targets, 4, ocfg)
    for ckpt in (True, False):
        m = copy.deepcopy(model)
        eng = FSDPEngine(m, ocfg, activation_checkpointing=ckpt)
        losses = [eng.step(tokens, targets).item() for _ in range(4)]
        for a, b in zip(losses, ref_losses):
            assert abs(a - b) < 2e-5, (ckpt, losses, ref_losses)
        state = eng.gather_full_state()
        for n, p in ref.named_parameters():
            assert torch.allclose(state[n], p.detach(), atol=2e-5), n


def test_engine_gradient_clipping_matches_clip_grad_norm():
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(num_layers=2)
    model = Llama(cfg)
    model.reset_parameters(0)
    ref = copy.deepcopy(model)
    tokens = torch.randint(0, cfg.vocab_size, (2, 24))
    targets = torch.randint(0, cfg.vocab_size, (2, 24))
    ocfg = AdamWConfig(lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    max_norm = 0.05  # well below the actual norm, so the clip is active
    opt = torch.optim.AdamW(ref.parameters(), lr=ocfg.lr, betas=ocfg.betas, eps=ocfg.eps, weight_decay=ocfg.weight_decay)
    norms = []
    for _ in range(3):
        opt.zero_grad()
        ref(tokens, targets).backward()
        norms.append(float(torch.nn.utils.clip_grad_norm_(ref.parameters(), max_norm)))
        opt.step()
    eng = FSDPEngine(copy.deepcopy(model), ocfg, max_grad_norm=max_norm)
    for i in range(3):
        eng.step(tokens, targets)
        assert abs(float(eng.grad_norm) - norms[i]) < 1e-4 * max(1.0, norms[i]), (i, float(eng.grad_norm), norms[i])
    assert norms[0] > max_norm
    state = eng.gather_full_state()
    for n, p in ref.named_parameters():
        assert torch.allclose(state[n], p.detach(), atol=3e-5), n


def test_selective_checkpointing_keeps_gemm_outputs_and_matches_autograd():
    from tensorplay_b200.ops import _ckpt
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(num_layers=2)
    model = Llama(cfg)
    model.reset_parameters(0)
    blk = model.layers[0]
    x = torch.randn(2, 24, cfg.hidden_size, requires_grad=True)
    extra = model.layer_extra_args(torch.zeros(2, 24, dtype=torch.long))
    y = blk(x, *extra)
    g = torch.randn_like(y)
    y.backward(g)
    ref = {n: p.grad.clone() for n, p in blk.named_parameters()}
    rx = x.grad.clone()
    for p in blk.parameters():
        p.grad = None
    x.grad = None
    with torch.no_grad(), _ckpt.record() as kept:
        blk(x.detach(), *extra)
    assert len(kept) == 4  # qkv, o_proj, gate_up, down projections (attention recomputes on CPU)
    with _ckpt.replay(kept):
        y2 = blk(x, *extra)
    y2.backward(g)
    torch.testing.assert_close(y2, y)
    torch.testing.assert_close(x.grad, rx)
    for n, p in blk.named_parameters():
        torch.testing.assert_close(p.grad, ref[n])
    # a replay that runs other ops than the record is an error, not a silent mismatch
    import pytest
    with pytest.raises(RuntimeError):
        with _ckpt.replay(kept[:2]):
            blk(x, *extra)
    # the engine produces the same training trajectory in all three modes
    tokens = torch.randint(0, cfg.vocab_size, (2, 24))
    losses = {}
    for mode in (True, "selective"):
        eng = FSDPEngine(copy.deepcopy(model), AdamWConfig(lr=1e-3), activation_checkpointing=mode)
        losses[mode] = [eng.step(tokens, tokens).item() for _ in range(3)]
    for a, b in zip(losses[True], losses["selective"]):
        assert abs(a - b) < 5e-4, losses
