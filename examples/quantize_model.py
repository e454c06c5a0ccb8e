"""Train a small decoder LM on a synthetic copy task, then compare post-training quantisation
recipes on it: plain int8 / int4 weight-only, activation-aware int4 (AWQ) and 2:4 pruning, by
perplexity, per-layer SQNR and greedy continuation.

    python examples/quantize_model.py [--steps 150]
"""
import argparse
import copy
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tensorplay_b200 import metrics, nn  # noqa: E402
from tensorplay_b200 import quantization as Q  # noqa: E402


def batches(vocab, n, seq, seed):
    """Sequences whose second half repeats the first: learnable, so perplexity means something."""
    g = torch.Generator().manual_seed(seed)
    half = torch.randint(2, vocab, (n, seq // 2), generator=g)
    return torch.cat((half, half), 1)


def perplexity(model, data):
    m = metrics.Perplexity()
    with torch.no_grad():
        m.update(model(data[:, :-1]), data[:, 1:])
    return float(m.compute())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=150)
    ap.add_argument("--hidden", type=int, default=128)
    a = ap.parse_args()
    torch.manual_seed(0)
    vocab, seq = 64, 32
    model = nn.DecoderLM(vocab, a.hidden, 2, 4, 2, intermediate_size=256)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-3)
    for step in range(a.steps):
        data = batches(vocab, 32, seq, step)
        loss = model(data[:, :-1], data[:, 1:])
        opt.zero_grad()
        loss.backward()
        opt.step()
    model.eval()
    held = batches(vocab, 64, seq, 10_000)
    calib = [batches(vocab, 16, seq, 20_000 + i)[:, :-1] for i in range(4)]
    keep_head = lambda m, name: name != "lm_head"   # noqa: E731
    recipes = {
        "int8 weight-only": lambda m: Q.quantize_(m, "int8_weight_only", filter_fn=keep_head),
        "int4 weight-only (g128)": lambda m: Q.quantize_(m, "int4_weight_only", group_size=128, filter_fn=keep_head),
        "int4 AWQ (g128)": lambda m: Q.awq_quantize_(m, calib, bits=4, group_size=128, filter_fn=keep_head),
        "2:4 pruned": lambda m: (lambda sp: (sp.step(), sp.squash()))(Q.WeightSparsifier(m, pattern=(2, 4),
                                                                                         filter_fn=keep_head)),
    }
    print(f"bf16/fp32 reference: perplexity {perplexity(model, held):.3f}")
    ref_gen = nn.generate(model, held[:2, : seq // 2 + 2], max_new_tokens=8)
    for name, apply in recipes.items():
        m = copy.deepcopy(model)
        apply(m)
        rep = Q.compare_models(model, m, calib[:1])
        worst = min(rep.values()) if rep else float("nan")
        same = bool(torch.equal(nn.generate(m, held[:2, : seq // 2 + 2], max_new_tokens=8), ref_gen))
        print(f"{name}: perplexity {perplexity(m, held):.3f}  worst layer SQNR {worst:.1f} dB  "
              f"greedy continuation unchanged: {same}")


if __name__ == "__main__":
    main()
