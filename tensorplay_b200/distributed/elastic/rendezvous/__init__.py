"""Elastic rendezvous: ``DynamicRendezvousHandler`` over this package's stores (own implementation
in ``dynamic.py``), timeouts, endpoint parsing, the store-backed state back end, the static handler and the handler
registry (``extras.py``); the etcd back ends and the parameter class resolve to PyTorch's module of the same role."""
from .dynamic import (DynamicRendezvousHandler, RendezvousClosedError, RendezvousSettings, RendezvousStateError,
                      RendezvousTimeoutError, create_handler)

from .extras import (P10dRendezvousBackend, RendezvousConnectionError, RendezvousError, RendezvousExhaustedError,  # noqa: F401
                     RendezvousGracefulExitError, RendezvousHandlerRegistry, RendezvousTimeout, StaticTCPRendezvous,
                     StoreRendezvousBackend, TpRendezvousBackend, _matches_machine_hostname, _parse_rendezvous_config,
                     _PeriodicTimer, get_registry, parse_rendezvous_endpoint, rendezvous_handler_registry)

__all__ = ["DynamicRendezvousHandler", "RendezvousSettings", "RendezvousClosedError", "RendezvousTimeoutError",
           "RendezvousStateError", "create_handler", "RendezvousTimeout", "RendezvousExhaustedError", "StaticTCPRendezvous",
           "StoreRendezvousBackend", "P10dRendezvousBackend", "TpRendezvousBackend", "get_registry",
           "parse_rendezvous_endpoint", "RendezvousHandlerRegistry"]


def __getattr__(name):
    import importlib
    for mod in ("torch.distributed.elastic.rendezvous", "torch.distributed.elastic.rendezvous.api"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
