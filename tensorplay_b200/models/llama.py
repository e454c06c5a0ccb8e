"""Llama-family decoder (RMSNorm, RoPE, grouped-query attention, SwiGLU) with packed QKV and
gate/up projections, so that a layer is four GEMMs plus row kernels.

Shapes follow the named configurations: Llama-3-8B (32 layers, hidden 4096, 32/8 heads of 128,
FFN 14336, vocab 128256, theta 5e5) and Llama-3-70B (80 layers, hidden 8192, 64/8 heads,
FFN 28672). The reference composes the same math from ``nn.GroupedQueryAttention`` /
``nn.SwiGLUMLP`` / ``nn.RMSNorm`` (tensorplay/nn/modules/causal_attention.py:30-187,
modern_block.py:29-103).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import Tensor, nn

from .. import ops


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_seq_len: int = 4096
    tie_embeddings: bool = False
    init_std: float = 0.02

    @staticmethod
    def llama3_8b(**kw) -> "LlamaConfig":
        return LlamaConfig(**kw)

    @staticmethod
    def llama3_70b(**kw) -> "LlamaConfig":
        return LlamaConfig(hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8,
                           ffn_size=28672, **kw)

    @staticmethod
    def tiny(**kw) -> "LlamaConfig":
        base = dict(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                    head_dim=64, ffn_size=512, max_seq_len=256)
        base.update(kw)
        return LlamaConfig(**base)

    def num_params(self) -> int:
        per_layer = (self.hidden_size * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
                     + self.num_heads * self.head_dim * self.hidden_size
                     + 3 * self.hidden_size * self.ffn_size + 2 * self.hidden_size)
        emb = self.vocab_size * self.hidden_size
        return self.num_layers * per_layer + emb * (1 if self.tie_embeddings else 2) + self.hidden_size

    def flops_per_token(self, seq_len: int, backward: bool = True, recompute: bool = False) -> float:
        """Model FLOPs per token: 2 * matmul params (+ causal attention), x3 with backward."""
        mm = self.num_params() - self.vocab_size * self.hidden_size * (0 if self.tie_embeddings else 1) \
            - self.hidden_size * (2 * self.num_layers + 1)
        fwd = 2.0 * mm + 2.0 * 2 * self.num_layers * self.num_heads * self.head_dim * seq_len / 2
        mult = 1.0 + (2.0 if backward else 0.0) + (1.0 if recompute else 0.0)
        return fwd * mult


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer_idx: int = 0, device=None, dtype=None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        H, D = cfg.hidden_size, cfg.head_dim
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.attn_norm = nn.Parameter(torch.ones(H, **kw))
        self.wqkv = nn.Parameter(torch.empty((cfg.num_heads + 2 * cfg.num_kv_heads) * D, H, **kw))
        self.wo = nn.Parameter(torch.empty(H, cfg.num_heads * D, **kw))
        self.ffn_norm = nn.Parameter(torch.ones(H, **kw))
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.ffn_size, H, **kw))
        self.w_down = nn.Parameter(torch.empty(H, cfg.ffn_size, **kw))

    def reset_parameters(self, generator=None) -> None:
        for w in (self.wqkv, self.wo, self.w_gate_up, self.w_down):
            nn.init.normal_(w, mean=0.0, std=self.cfg.init_std, generator=generator)
        nn.init.ones_(self.attn_norm)
        nn.init.ones_(self.ffn_norm)

    def forward(self, x: Tensor, cos: Tensor, sin: Tensor, position_ids: Optional[Tensor] = None,
                past_key_values=None) -> Tensor:
        cfg = self.cfg
        h = ops.rms_norm(x, self.attn_norm, cfg.rms_eps)
        qkv = ops.linear(h, self.wqkv)
        if past_key_values is None:
            a = ops.qkv_attention(qkv, cos, sin, position_ids, cfg.num_heads, cfg.num_kv_heads,
                                  cfg.head_dim, causal=True)
        else:
            a = self._attend_cached(qkv, cos, sin, position_ids, past_key_values)
        a = ops.linear(a, self.wo)
        h, x = ops.rms_norm(a, self.ffn_norm, cfg.rms_eps, residual=x)
        gu = ops.linear(h, self.w_gate_up)
        return x + ops.linear(ops.swiglu_packed(gu), self.w_down)

    def _attend_cached(self, qkv, cos, sin, position_ids, cache):
        cfg = self.cfg
        B, T, _ = qkv.shape
        Hq, Hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        packed = qkv.view(B, T, Hq + 2 * Hkv, D)
        off = cache.get_seq_length(self.layer_idx)
        pos = position_ids
        if pos is None and off:
            pos = torch.arange(off, off + T, device=qkv.device).expand(B, T)
        qk = ops.apply_rope(packed[:, :, : Hq + Hkv], cos, sin, pos)
        k, v = cache.update(qk[:, :, Hq:].transpose(1, 2), packed[:, :, Hq + Hkv:].transpose(1, 2),
                            self.layer_idx)
        o = ops.flash_attention(qk[:, :, :Hq], k.transpose(1, 2), v.transpose(1, 2), causal=True)
        return o.reshape(B, T, Hq * D)


class Llama(nn.Module):
    """Decoder-only LM. ``forward(tokens, targets=None)`` returns logits, or the mean
    next-token loss when ``targets`` is given."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.cfg = cfg
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList([LlamaBlock(cfg, i, **kw) for i in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, **kw))
        if cfg.tie_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self._rope = None

    def reset_parameters(self, seed: Optional[int] = None) -> None:
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.embed.device)
            gen.manual_seed(seed)
        nn.init.normal_(self.embed, std=self.cfg.init_std, generator=gen)
        if self.lm_head is not None:
            nn.init.normal_(self.lm_head, std=self.cfg.init_std, generator=gen)
        nn.init.ones_(self.final_norm)
        for layer in self.layers:
            layer.reset_parameters(gen)

    def rope_tables(self, n: int, device):
        if self._rope is None or self._rope[0].shape[0] < n or self._rope[0].device != torch.device(device):
            self._rope = ops.rope_tables(max(n, self.cfg.max_seq_len), self.cfg.head_dim,
                                         self.cfg.rope_theta, device=device)
        return self._rope

    def layer_extra_args(self, tokens: Tensor):
        """Per-step arguments every block receives after the hidden states (RoPE tables)."""
        return self.rope_tables(tokens.shape[1], tokens.device)

    def create_empty_cache(self):
        from ..nn.cache import DynamicCache
        return DynamicCache()

    def embed_tokens(self, tokens: Tensor) -> Tensor:
        return _embedding(tokens, self.embed)

    def head(self, x: Tensor, targets: Optional[Tensor] = None) -> Tensor:
        h = ops.rms_norm(x, self.final_norm, self.cfg.rms_eps)
        w = self.embed if self.lm_head is None else self.lm_head
        logits = ops.linear(h, w)
        if targets is None:
            return logits
        return ops.cross_entropy(logits.view(-1, logits.shape[-1]), targets.reshape(-1))

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None,
                position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        B, T = tokens.shape
        off = past_key_values.get_seq_length(0) if past_key_values is not None else 0
        cos, sin = self.rope_tables(off + T, tokens.device)
        x = self.embed_tokens(tokens)
        for layer in self.layers:
            x = layer(x, cos, sin, position_ids, past_key_values)
        return self.head(x, targets)


def _embedding(tokens: Tensor, weight: Tensor) -> Tensor:
    """Row gather; the backward scatter-adds straight into the weight's gradient buffer."""
    return ops.embedding(tokens, weight)
