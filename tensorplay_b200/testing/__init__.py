"""``testing``: ``assert_close`` / ``make_tensor`` (tensorplay/testing/_comparison.py, _creation.py)."""
from torch.testing import assert_close, make_tensor  # noqa: F401

__all__ = ["assert_close", "make_tensor"]


def __getattr__(name):
    """Comparison helpers resolve to PyTorch's testing package."""
    import importlib
    for mod in ['torch.testing', 'torch.testing._comparison', 'torch.testing._internal.common_utils']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def assert_allclose(actual, expected, rtol=None, atol=None, equal_nan: bool = True, msg: str = "") -> None:
    """Older spelling of ``assert_close`` (dtype-based default tolerances, NaNs equal by default)."""
    import torch
    torch.testing.assert_close(torch.as_tensor(actual), torch.as_tensor(expected), rtol=rtol, atol=atol,
                               equal_nan=equal_nan, check_dtype=False, msg=msg or None)


def default_tolerances(*inputs):
    """``(rtol, atol)`` used by ``assert_close`` for the widest dtype among ``inputs`` (tensors or dtypes)."""
    import torch
    from torch.testing._comparison import default_tolerances as _dt
    return _dt(*[i if isinstance(i, torch.dtype) else i.dtype for i in inputs])


def get_tolerances(*inputs, rtol=None, atol=None):
    if rtol is not None and atol is not None:
        return rtol, atol
    return default_tolerances(*inputs)
