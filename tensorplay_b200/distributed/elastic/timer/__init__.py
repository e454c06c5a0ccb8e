"""Expiration timers for worker code: the file-based local timer is implemented here
(``file_based_local_timer.py``); the other names resolve to PyTorch's module of the same role."""
from .file_based_local_timer import FileTimerClient, FileTimerRequest, FileTimerServer, configure, expires

__all__ = ["FileTimerClient", "FileTimerRequest", "FileTimerServer", "configure", "expires"]


def __getattr__(name):
    import importlib
    try:
        return getattr(importlib.import_module("torch.distributed.elastic.timer"), name)
    except (ImportError, AttributeError):
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
