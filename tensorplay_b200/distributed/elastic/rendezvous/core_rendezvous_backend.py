"""Import path of the store-backed rendezvous state back end (one implementation under the reference's three module
names: ``p10d_``, ``core_`` and ``tp_rendezvous_backend``)."""
from .extras import P10dRendezvousBackend, StoreRendezvousBackend, TpRendezvousBackend  # noqa: F401

CoreRendezvousBackend = StoreRendezvousBackend


def create_backend(store, run_id: str):
    """``(backend, store)`` as the dynamic handler's factory expects."""
    return StoreRendezvousBackend(store, run_id), store
