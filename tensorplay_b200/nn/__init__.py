"""``nn``: torch.nn's module zoo plus the LLM stack of the reference computed by sm_100a kernels."""
from torch.nn import *  # noqa: F401,F403
from torch.nn import Module, Parameter, init, utils  # noqa: F401
import torch.nn as _tnn

import importlib as _importlib

# ``from torch.nn import *`` above has already bound ``functional``, ``attention``, ``parallel`` and
# ``modules`` to torch's sub-packages, and ``from . import x`` keeps an existing attribute: this
# package's own sub-modules of those names are imported by path and bound explicitly.
functional = _importlib.import_module(__name__ + ".functional")
attention = _importlib.import_module(__name__ + ".attention")
modules = _importlib.import_module(__name__ + ".modules")
from . import cache, generation  # noqa: F401,E402
from .cache import (Cache, DynamicCache, LinearStateCache, PagedCache, QuantizedCache,
                    SlidingWindowCache, StaticCache)
from .generation import generate, sample, top_k_top_p_filtering
from .modules import (DecoderLM, CausalEncoderDecoder, CompressedSparseAttention, CrossAttention, GatedDeltaNet, GroupedQueryAttention, KimiDeltaAttention, LayerNorm, Linear,
                      MultiheadLatentAttention, RMSNorm, RotaryEmbedding, SwiGLUMLP, TransformerBlock,
                      apply_rotary_emb, chunk_gated_delta_rule, gated_delta_rule)
from .modules import (DepthwiseConv2d, GatedRMSNorm, chunk_kimi_delta_rule, recurrent_gated_delta_rule,  # noqa: E402
                      recurrent_kimi_delta_rule)
parallel = _importlib.import_module(__name__ + ".parallel")


def __getattr__(name):
    return getattr(_tnn, name)
