"""``backends``: PyTorch's backend switches (``cudnn``, ``cuda.matmul`` ...); ``backends.cuda`` adds the queries the
reference lists there (tensorplay/backends/cuda/__init__.py)."""
from . import cuda  # noqa: F401


def __getattr__(name):
    import importlib
    import torch.backends as _b
    try:
        return getattr(_b, name)
    except AttributeError:
        try:
            return importlib.import_module(f"torch.backends.{name}")
        except ImportError:
            raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
