"""Attention-bias objects (``causal_upper_left``, ``causal_lower_right``, ``CausalBias``): PyTorch's."""
from torch.nn.attention.bias import *  # noqa: F401,F403
from torch.nn.attention.bias import CausalBias, CausalVariant, causal_lower_right, causal_upper_left  # noqa: F401
