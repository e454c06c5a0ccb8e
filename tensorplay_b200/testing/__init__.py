"""``testing``: ``assert_close`` / ``make_tensor`` (tensorplay/testing/_comparison.py, _creation.py)."""
from torch.testing import assert_close, make_tensor  # noqa: F401

__all__ = ["assert_close", "make_tensor"]
