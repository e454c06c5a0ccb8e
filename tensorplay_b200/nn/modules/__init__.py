from .llm import (GroupedQueryAttention, LayerNorm, Linear, RMSNorm, RotaryEmbedding, SwiGLUMLP,
                  TransformerBlock, apply_rotary_emb)

from .lm import DecoderLM
from .mixers import (CausalEncoderDecoder, CompressedSparseAttention, CrossAttention, GatedDeltaNet, KimiDeltaAttention, MultiheadLatentAttention, chunk_gated_delta_rule,
                     gated_delta_rule)

__all__ = ["GroupedQueryAttention", "LayerNorm", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLUMLP",
           "TransformerBlock", "apply_rotary_emb", "MultiheadLatentAttention", "GatedDeltaNet", "gated_delta_rule",
           "chunk_gated_delta_rule", "KimiDeltaAttention", "CrossAttention", "CausalEncoderDecoder", "CompressedSparseAttention", "DecoderLM"]

from ... import _views as _views  # noqa: E402

# the reference's one-class-per-file module names (nn.modules.gated_delta, .rotary, .modern_block ...)
_views.install(__name__, max_depth=1, namespace=__name__.rsplit(".", 1)[0])
