from .llm import (GroupedQueryAttention, LayerNorm, Linear, RMSNorm, RotaryEmbedding, SwiGLUMLP,
                  TransformerBlock, apply_rotary_emb)

__all__ = ["GroupedQueryAttention", "LayerNorm", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLUMLP",
           "TransformerBlock", "apply_rotary_emb"]
