from .llm import (GroupedQueryAttention, LayerNorm, Linear, RMSNorm, RotaryEmbedding, SwiGLUMLP,
                  TransformerBlock, apply_rotary_emb)

from .lm import DecoderLM
from .mixers import (CausalEncoderDecoder, CompressedSparseAttention, CrossAttention, GatedDeltaNet, KimiDeltaAttention, MultiheadLatentAttention, chunk_gated_delta_rule,
                     gated_delta_rule)

__all__ = ["GroupedQueryAttention", "LayerNorm", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLUMLP",
           "TransformerBlock", "apply_rotary_emb", "MultiheadLatentAttention", "GatedDeltaNet", "gated_delta_rule",
           "chunk_gated_delta_rule", "KimiDeltaAttention", "CrossAttention", "CausalEncoderDecoder", "CompressedSparseAttention", "DecoderLM"]
