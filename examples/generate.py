"""Autoregressive generation with the ``nn`` LLM stack: a small decoder built from
``TransformerBlock`` + ``GroupedQueryAttention`` with a KV cache, sampled with ``nn.generate``.

    python examples/generate.py --new-tokens 32 --top-k 40 --top-p 0.9 --cache static

Random-init weights (no network for checkpoints); pass ``--load weights.mega`` for a trained
state dict saved with ``tensorplay_b200.save``.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import tensorplay_b200 as tp  # noqa: E402
from tensorplay_b200 import nn  # noqa: E402


class TinyLM(nn.Module):
    def __init__(self, vocab=512, hidden=128, layers=2, heads=4, kv_heads=2, max_len=256, cache="dynamic"):
        super().__init__()
        self.embed = nn.Embedding(vocab, hidden)
        self.blocks = nn.ModuleList(
            nn.TransformerBlock(hidden, nn.GroupedQueryAttention(hidden, heads, num_kv_heads=kv_heads, layer_idx=i))
            for i in range(layers))
        self.norm = nn.RMSNorm(hidden)
        self.head = nn.Linear(hidden, vocab, bias=False)
        self.max_len, self.cache_kind = max_len, cache

    def create_empty_cache(self):
        return {"dynamic": nn.DynamicCache, "static": lambda: nn.StaticCache(self.max_len),
                "paged": lambda: nn.PagedCache(block_size=16)}[self.cache_kind]()

    def forward(self, input_ids, position_ids=None, past_key_values=None):
        x = self.embed(input_ids)
        for b in self.blocks:
            x = b(x, position_ids=position_ids, past_key_values=past_key_values)
        return self.head(self.norm(x))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--cache", default="dynamic", choices=["dynamic", "static", "paged"])
    ap.add_argument("--load", default=None)
    args = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    torch.manual_seed(0)
    model = TinyLM(cache=args.cache).to(dev)
    if dev == "cuda":
        model = model.bfloat16()
    if args.load:
        model.load_state_dict(tp.load(args.load))
    model.eval()
    prompt = torch.randint(0, 512, (2, 8), device=dev)
    out = nn.generate(model, prompt, max_new_tokens=args.new_tokens, do_sample=True, temperature=args.temperature,
                      top_k=args.top_k, top_p=args.top_p)
    greedy = nn.generate(model, prompt, max_new_tokens=args.new_tokens)
    nocache = nn.generate(model, prompt, max_new_tokens=args.new_tokens, use_cache=False)
    print("sampled:", out[0].tolist())
    print("greedy :", greedy[0].tolist())
    print("greedy with and without cache agree:", bool((greedy == nocache).all()))


if __name__ == "__main__":
    main()
