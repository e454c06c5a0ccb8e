"""GPT-2-family decoder (LayerNorm, learned positions, GELU MLP, tied embeddings).

Covers the GPT-2-small training configuration (12 layers, d=768, 12 heads, MLP 3072, vocab 50257,
context 1024) and the CPU toy LLM (2 layers, d=128, 4 heads, vocab 512, context 64).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import Tensor, nn

from .. import ops
from .llama import _embedding


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_ctx: int = 1024
    d_model: int = 768
    n_layers: int = 12
    n_heads: int = 12
    mlp_ratio: int = 4
    ln_eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = True
    gelu_approximate: str = "tanh"

    @staticmethod
    def small(**kw) -> "GPT2Config":
        return GPT2Config(**kw)

    @staticmethod
    def toy(**kw) -> "GPT2Config":
        base = dict(vocab_size=512, n_ctx=64, d_model=128, n_layers=2, n_heads=4)
        base.update(kw)
        return GPT2Config(**base)

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 127) // 128 * 128


class GPT2Block(nn.Module):
    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        d = cfg.d_model
        self.cfg = cfg
        self.ln1_w = nn.Parameter(torch.ones(d, **kw))
        self.ln1_b = nn.Parameter(torch.zeros(d, **kw))
        self.w_qkv = nn.Parameter(torch.empty(3 * d, d, **kw))
        self.b_qkv = nn.Parameter(torch.zeros(3 * d, **kw))
        self.w_o = nn.Parameter(torch.empty(d, d, **kw))
        self.b_o = nn.Parameter(torch.zeros(d, **kw))
        self.ln2_w = nn.Parameter(torch.ones(d, **kw))
        self.ln2_b = nn.Parameter(torch.zeros(d, **kw))
        self.w_fc = nn.Parameter(torch.empty(cfg.mlp_ratio * d, d, **kw))
        self.b_fc = nn.Parameter(torch.zeros(cfg.mlp_ratio * d, **kw))
        self.w_proj = nn.Parameter(torch.empty(d, cfg.mlp_ratio * d, **kw))
        self.b_proj = nn.Parameter(torch.zeros(d, **kw))

    def reset_parameters(self, generator=None):
        for w in (self.w_qkv, self.w_o, self.w_fc, self.w_proj):
            nn.init.normal_(w, std=self.cfg.init_std, generator=generator)

    def forward(self, x: Tensor) -> Tensor:
        cfg = self.cfg
        B, T, d = x.shape
        H = cfg.n_heads
        h = ops.layer_norm(x, self.ln1_w, self.ln1_b, cfg.ln_eps)
        qkv = ops.linear(h, self.w_qkv, self.b_qkv).view(B, T, 3, H, d // H)
        a = ops.flash_attention(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], causal=True)
        x = x + ops.linear(a.reshape(B, T, d), self.w_o, self.b_o)
        h = ops.layer_norm(x, self.ln2_w, self.ln2_b, cfg.ln_eps)
        h = ops.gelu(ops.linear(h, self.w_fc, self.b_fc), cfg.gelu_approximate)
        return x + ops.linear(h, self.w_proj, self.b_proj)


class GPT2(nn.Module):
    embed_param_names = ("wte", "wpe")

    def __init__(self, cfg: GPT2Config, device=None, dtype=None):
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg = cfg
        # the embedding table is padded to a multiple of 128 rows so that the tied LM head is a
        # tile-aligned GEMM; padded logits are masked out of the loss
        self.wte = nn.Parameter(torch.empty(cfg.padded_vocab, cfg.d_model, **kw))
        self.wpe = nn.Parameter(torch.empty(cfg.n_ctx, cfg.d_model, **kw))
        self.layers = nn.ModuleList([GPT2Block(cfg, **kw) for _ in range(cfg.n_layers)])
        self.lnf_w = nn.Parameter(torch.ones(cfg.d_model, **kw))
        self.lnf_b = nn.Parameter(torch.zeros(cfg.d_model, **kw))
        self._pad_bias = None  # constant epilogue bias that masks the padded vocabulary columns
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.padded_vocab, cfg.d_model, **kw))

    def reset_parameters(self, seed: Optional[int] = None) -> None:
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.wte.device)
            gen.manual_seed(seed)
        nn.init.normal_(self.wte, std=self.cfg.init_std, generator=gen)
        nn.init.normal_(self.wpe, std=self.cfg.init_std, generator=gen)
        with torch.no_grad():
            self.wte[self.cfg.vocab_size:].zero_()
        if self.lm_head is not None:
            nn.init.normal_(self.lm_head, std=self.cfg.init_std, generator=gen)
        for l in self.layers:
            l.reset_parameters(gen)

    def embed_tokens(self, tokens: Tensor) -> Tensor:
        T = tokens.shape[1]
        return _embedding(tokens, self.wte) + self.wpe[:T]

    def head(self, x: Tensor, targets: Optional[Tensor] = None) -> Tensor:
        h = ops.layer_norm(x, self.lnf_w, self.lnf_b, self.cfg.ln_eps)
        w = self.wte if self.lm_head is None else self.lm_head
        V = self.cfg.vocab_size
        if targets is not None and h.is_cuda and h.dtype == torch.bfloat16:
            # padded vocabulary columns hold exactly-zero weights; a constant bias in the GEMM
            # epilogue pushes them out of the softmax without another pass over the logits
            if self._pad_bias is None or self._pad_bias.device != h.device:
                pb = torch.zeros(w.shape[0], dtype=torch.bfloat16, device=h.device)
                pb[V:] = -30000.0
                self._pad_bias = pb
            logits = ops.linear(h, w, self._pad_bias)
            return ops.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1))
        logits = ops.linear(h, w)
        if targets is None:
            return logits[..., :V]
        return ops.cross_entropy(logits[..., :V].reshape(-1, V), targets.reshape(-1))

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None, position_ids=None,
                past_key_values=None) -> Tensor:
        x = self.embed_tokens(tokens)
        for layer in self.layers:
            x = layer(x)
        return self.head(x, targets)
