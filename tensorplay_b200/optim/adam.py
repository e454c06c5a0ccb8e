"""``optim.adam``: the fused Adam of this framework (tensorplay/optim/adam.py:27-520)."""
from .adamw import Adam, AdamW  # noqa: F401
