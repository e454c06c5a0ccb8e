"""Expiration timers for worker code: the file-based local timer is implemented here
(``file_based_local_timer.py``); the other names resolve to PyTorch's module of the same role."""
from .file_based_local_timer import FileTimerClient, FileTimerRequest, FileTimerServer, configure, expires

__all__ = ["FileTimerClient", "FileTimerRequest", "FileTimerServer", "configure", "expires"]


def __getattr__(name):
    import importlib
    for mod in ("torch.distributed.elastic.timer", "torch.distributed.elastic.timer.api",
                "torch.distributed.elastic.timer.local_timer", "torch.distributed.elastic.timer.file_based_local_timer"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    if name == "FileTimerRequestQueue":          # the file-based server reads its pipe itself: the queue is its private part
        from .file_based_local_timer import FileTimerServer
        return FileTimerServer
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
