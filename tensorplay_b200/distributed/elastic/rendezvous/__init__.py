"""Elastic rendezvous: ``DynamicRendezvousHandler`` over this package's stores (own implementation
in ``dynamic.py``); the registry, the parameter class and the other handler names resolve to
PyTorch's module of the same role."""
from .dynamic import (DynamicRendezvousHandler, RendezvousClosedError, RendezvousSettings, RendezvousStateError,
                      RendezvousTimeoutError, create_handler)

__all__ = ["DynamicRendezvousHandler", "RendezvousSettings", "RendezvousClosedError", "RendezvousTimeoutError",
           "RendezvousStateError", "create_handler"]


def __getattr__(name):
    import importlib
    for mod in ("torch.distributed.elastic.rendezvous", "torch.distributed.elastic.rendezvous.api"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
