"""A decoder language model assembled from the module-level LLM stack (embedding, pre-norm blocks
with grouped-query attention and SwiGLU, final norm, LM head). Every projection is an ``nn.Linear``,
so module-level tools apply to it directly: ``quantization.quantize_`` / ``awq_quantize_``, the
sparsifier, ``fully_shard``, the tensor-parallel styles, ``lumen`` layer attributions."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor
from torch.nn import Embedding, Module, ModuleList

from .llm import GroupedQueryAttention, Linear, RMSNorm, TransformerBlock


class DecoderLM(Module):
    def __init__(self, vocab_size: int, hidden_size: int, num_layers: int, num_heads: int,
                 num_kv_heads: Optional[int] = None, intermediate_size: Optional[int] = None,
                 rope_base: float = 10000.0, rms_norm_eps: float = 1e-6, tie_embeddings: bool = False,
                 device=None, dtype=None) -> None:
        super().__init__()
        kw = {"device": device, "dtype": dtype}
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.embed = Embedding(vocab_size, hidden_size, **kw)
        self.layers = ModuleList([
            TransformerBlock(hidden_size,
                             GroupedQueryAttention(hidden_size, num_heads, num_kv_heads, rope_base=rope_base,
                                                   rms_norm_eps=rms_norm_eps, layer_idx=i, **kw),
                             mlp_intermediate_size=intermediate_size, rms_norm_eps=rms_norm_eps, **kw)
            for i in range(num_layers)])
        self.norm = RMSNorm(hidden_size, eps=rms_norm_eps, **kw)
        self.lm_head = Linear(hidden_size, vocab_size, bias=False, **kw)
        if tie_embeddings:
            self.lm_head.weight = self.embed.weight

    def create_empty_cache(self):
        from ..cache import DynamicCache
        return DynamicCache()

    def hidden_states(self, tokens: Tensor, position_ids: Optional[Tensor] = None, past_key_values=None) -> Tensor:
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x, position_ids=position_ids, past_key_values=past_key_values)
        return self.norm(x)

    def forward(self, tokens: Tensor, targets: Optional[Tensor] = None, position_ids: Optional[Tensor] = None,
                past_key_values=None) -> Tensor:
        """Logits ``[B, T, V]``, or the mean next-token cross-entropy when ``targets`` is given."""
        logits = self.lm_head(self.hidden_states(tokens, position_ids, past_key_values))
        if targets is None:
            return logits
        return torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
