from .llm import (GroupedQueryAttention, LayerNorm, Linear, RMSNorm, RotaryEmbedding, SwiGLUMLP,
                  TransformerBlock, apply_rotary_emb)

from .lm import DecoderLM
from .mixers import (CausalEncoderDecoder, CompressedSparseAttention, CrossAttention, DepthwiseConv2d, GatedDeltaNet,
                     GatedRMSNorm, KimiDeltaAttention, MultiheadLatentAttention, chunk_gated_delta_rule,
                     chunk_kimi_delta_rule, gated_delta_rule, recurrent_gated_delta_rule, recurrent_kimi_delta_rule)

__all__ = ["GroupedQueryAttention", "LayerNorm", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLUMLP",
           "TransformerBlock", "apply_rotary_emb", "MultiheadLatentAttention", "GatedDeltaNet", "gated_delta_rule",
           "chunk_gated_delta_rule", "KimiDeltaAttention", "CrossAttention", "CausalEncoderDecoder", "CompressedSparseAttention", "DecoderLM", "GatedRMSNorm", "DepthwiseConv2d",
           "recurrent_gated_delta_rule", "recurrent_kimi_delta_rule", "chunk_kimi_delta_rule"]

def __getattr__(name):
    """The long tail of layers (``Conv2d``, ``BatchNorm1d``, ``LSTM`` ...) is PyTorch's."""
    import torch.nn as _nn
    for ns in (_nn.modules, _nn, _nn.modules.linear, _nn.modules.activation):
        try:
            return getattr(ns, name)
        except AttributeError:
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


from ... import _views as _views  # noqa: E402

# the reference's one-class-per-file module names (nn.modules.gated_delta, .rotary, .modern_block ...)
_views.install(__name__, max_depth=1, namespace=__name__.rsplit(".", 1)[0],
               names=("latent_attention", "multihead_attention", "kimi_delta", "compressed_attention", "gated_delta",
                      "causal_attention", "causal_encoder_decoder", "folding", "modern_block", "rotary"))
