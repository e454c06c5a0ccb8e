"""``nn``: torch.nn's module zoo plus the LLM stack of the reference computed by sm_100a kernels."""
from torch.nn import *  # noqa: F401,F403
from torch.nn import Module, Parameter, init, utils  # noqa: F401
import torch.nn as _tnn

from . import cache, functional, generation  # noqa: F401
from .cache import (Cache, DynamicCache, LinearStateCache, PagedCache, QuantizedCache,
                    SlidingWindowCache, StaticCache)
from .generation import generate, sample, top_k_top_p_filtering
from .modules import (DecoderLM, CausalEncoderDecoder, CompressedSparseAttention, CrossAttention, GatedDeltaNet, GroupedQueryAttention, KimiDeltaAttention, LayerNorm, Linear,
                      MultiheadLatentAttention, RMSNorm, RotaryEmbedding, SwiGLUMLP, TransformerBlock,
                      apply_rotary_emb, chunk_gated_delta_rule, gated_delta_rule)
from . import parallel  # noqa: F401,E402


def __getattr__(name):
    return getattr(_tnn, name)
