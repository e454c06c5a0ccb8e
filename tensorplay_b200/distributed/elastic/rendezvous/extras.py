"""The rest of the rendezvous surface (tensorplay/distributed/elastic/rendezvous/{api,utils,registry,
static_tcp_rendezvous,p10d_rendezvous_backend}.py): timeouts, endpoint / configuration parsing, a periodic timer,
the store-backed state back end with compare-and-set fencing, the static handler (ranks given by the launcher, one
TCP store), and a registry of handler factories keyed by back-end name."""
from __future__ import annotations

import ipaddress
import socket
import threading
from datetime import timedelta
from typing import Any, Callable, Dict, Optional, Tuple

from .dynamic import DynamicRendezvousHandler, RendezvousSettings, RendezvousStateError, RendezvousTimeoutError


class RendezvousError(Exception):
    pass


class RendezvousConnectionError(RendezvousError):
    pass


class RendezvousGracefulExitError(RendezvousError):
    pass


class RendezvousExhaustedError(RendezvousError):
    """No slot left: ``max_nodes`` nodes already form the job."""


class RendezvousTimeout:
    """The four time limits of a rendezvous; unspecified ones take their defaults."""

    _DEFAULTS = {"join": timedelta(seconds=600), "last_call": timedelta(seconds=30), "close": timedelta(seconds=30),
                 "heartbeat": timedelta(seconds=5)}

    def __init__(self, join: Optional[timedelta] = None, last_call: Optional[timedelta] = None,
                 close: Optional[timedelta] = None, heartbeat: Optional[timedelta] = None):
        for name, value in (("join", join), ("last_call", last_call), ("close", close), ("heartbeat", heartbeat)):
            value = self._DEFAULTS[name] if value is None else value
            if value <= timedelta(0):
                raise ValueError(f"The {name} timeout ({value}) must be positive.")
            setattr(self, "_" + name, value)

    join = property(lambda self: self._join)
    last_call = property(lambda self: self._last_call)
    close = property(lambda self: self._close)
    heartbeat = property(lambda self: self._heartbeat)


def _parse_rendezvous_config(config_str: str) -> Dict[str, str]:
    """``"k1=v1,k2=v2"`` -> dict; a key without ``=`` or an empty key or value is an error."""
    out: Dict[str, str] = {}
    config_str = config_str.strip()
    if not config_str:
        return out
    for pair in config_str.split(","):
        key, sep, value = pair.partition("=")
        key, value = key.strip(), value.strip()
        if not sep or not key or not value:
            raise ValueError("The rendezvous configuration string must be in format <key1>=<value1>,...,<keyN>=<valueN>.")
        out[key] = value
    return out


def parse_rendezvous_endpoint(endpoint: Optional[str], default_port: int) -> Tuple[str, int]:
    """``"host:port"`` / ``"host"`` / ``"[v6]:port"`` -> (host, port); no endpoint means this machine."""
    endpoint = (endpoint or "").strip()
    if not endpoint:
        return "localhost", default_port
    if endpoint.startswith("["):                                  # bracketed IPv6
        host, _, rest = endpoint[1:].partition("]")
        port = rest[1:] if rest.startswith(":") else ""
    elif endpoint.count(":") > 1:                                  # bare IPv6, no port
        host, port = endpoint, ""
    else:
        host, _, port = endpoint.partition(":")
    if port:
        if not port.isdigit() or not 0 < int(port) < 65536:
            raise ValueError(f"The port number of the rendezvous endpoint '{endpoint}' must be an integer between 0 and 65536.")
        port_n = int(port)
    else:
        port_n = default_port
    if not host or any(c.isspace() for c in host):
        raise ValueError(f"The hostname of the rendezvous endpoint '{endpoint}' must be a dot-separated list of labels, an IPv4 address, or an IPv6 address.")
    return host, port_n


def _matches_machine_hostname(host: str) -> bool:
    """Does ``host`` name this machine (loopback, its host name, or one of its addresses)?"""
    if host in ("localhost", socket.gethostname(), socket.getfqdn()):
        return True
    try:
        addr = ipaddress.ip_address(host)
    except ValueError:
        addr = None
    if addr is not None and addr.is_loopback:
        return True
    try:
        mine = {info[4][0] for info in socket.getaddrinfo(socket.gethostname(), None)}
    except OSError:
        mine = set()
    if addr is not None:
        return str(addr) in mine
    try:
        theirs = {info[4][0] for info in socket.getaddrinfo(host, None)}
    except OSError:
        return False
    return bool(theirs & (mine | {"127.0.0.1", "::1"}))


class _PeriodicTimer:
    """Calls ``function(*args, **kwargs)`` every ``interval`` on a daemon thread until cancelled."""

    def __init__(self, interval: timedelta, function: Callable[..., None], *args: Any, **kwargs: Any):
        self._interval, self._fn, self._args, self._kwargs = interval.total_seconds(), function, args, kwargs
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._name: Optional[str] = None

    def set_name(self, name: str) -> None:
        if self._thread is not None:
            raise RuntimeError("The timer has already started.")
        self._name = name

    def start(self) -> None:
        if self._thread is not None:
            raise RuntimeError("The timer has already started.")

        def loop():
            while not self._stop.wait(self._interval):
                self._fn(*self._args, **self._kwargs)
        self._thread = threading.Thread(target=loop, name=self._name or "PeriodicTimer", daemon=True)
        self._thread.start()

    def cancel(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join()


class StoreRendezvousBackend:
    """Keeps the rendezvous state as one value of a store; ``set_state`` only writes over the state whose token the
    caller holds (compare-and-set), so concurrent writers cannot lose each other's updates."""

    def __init__(self, store, run_id: str):
        self._store, self._key = store, f"tensorplay.rendezvous.{run_id}"

    @property
    def name(self) -> str:
        return "store"

    def get_state(self) -> Optional[Tuple[bytes, Any]]:
        if not self._store.check([self._key]):
            return None
        raw = self._store.get(self._key)
        return (raw, raw) if raw else None

    def set_state(self, state: bytes, token: Any = None) -> Optional[Tuple[bytes, Any, bool]]:
        expected = token if isinstance(token, (bytes, bytearray)) else b""
        got = self._store.compare_set(self._key, expected, state)
        return got, got, got == state


P10dRendezvousBackend = TpRendezvousBackend = StoreRendezvousBackend


class StaticTCPRendezvous:
    """Ranks are given (by the launcher): the rendezvous is one TCP store hosted by rank 0, nothing to negotiate."""

    def __init__(self, master_addr: str, master_port: int, rank: int, world_size: int, run_id: str, timeout: int = 300):
        self.master_addr, self.master_port = master_addr, master_port
        self.rank, self.world_size, self.run_id, self.timeout = rank, world_size, run_id, timeout
        self._store = None

    def get_backend(self) -> str:
        return "static"

    def next_rendezvous(self):
        from ...store import PrefixStore, TCPStore
        if self._store is None:
            self._store = TCPStore(self.master_addr, self.master_port, world_size=self.world_size,
                                   is_master=self.rank == 0, timeout=self.timeout)
        return PrefixStore(self.run_id, self._store), self.rank, self.world_size

    def is_closed(self) -> bool:
        return False

    def set_closed(self) -> None:
        pass

    def num_nodes_waiting(self) -> int:
        return 0

    def get_run_id(self) -> str:
        return self.run_id

    def shutdown(self) -> bool:
        return True


class RendezvousHandlerRegistry:
    def __init__(self):
        self._creators: Dict[str, Callable[..., Any]] = {}

    def register(self, backend: str, creator: Callable[..., Any]) -> None:
        if not backend:
            raise ValueError("The rendezvous backend name must be a non-empty string.")
        if backend in self._creators and self._creators[backend] is not creator:
            raise ValueError(f"The rendezvous backend '{backend}' cannot be registered twice with different creators.")
        self._creators[backend] = creator

    def create_handler(self, backend: str, *args, **kwargs):
        try:
            creator = self._creators[backend]
        except KeyError:
            raise ValueError(f"The rendezvous backend '{backend}' is not registered. Did you forget to call `register`?") from None
        return creator(*args, **kwargs)

    def backends(self):
        return sorted(self._creators)


_registry = RendezvousHandlerRegistry()
_registry.register("static", StaticTCPRendezvous)
_registry.register("dynamic", lambda store, run_id, min_nodes, max_nodes, **kw: DynamicRendezvousHandler(
    store, RendezvousSettings(run_id, min_nodes, max_nodes, **kw)))


def get_registry() -> RendezvousHandlerRegistry:
    return _registry


rendezvous_handler_registry = _registry
