"""Helpers of the elastic package (tensorplay/distributed/elastic/utils/{api,store,distributed}.py): environment
and socket helpers, the launcher's argument macros, and multi-key store operations with a deadline - ``get_all``,
``synchronize`` (every rank publishes a blob and reads all of them), ``barrier``."""
from __future__ import annotations

import contextlib
import os
import socket
from datetime import timedelta
from typing import Iterable, List, Optional, Union


def get_logger(name=None):
    """Logger named after the calling module (or ``name``), at the level in ``LOGLEVEL`` (default WARNING)."""
    import logging
    import sys as _sys
    if name is None:
        name = _sys._getframe(1).f_globals.get("__name__", "tensorplay_b200.distributed.elastic")
    log = logging.getLogger(name)
    log.setLevel(os.environ.get("LOGLEVEL", "WARNING"))
    return log


def get_env_variable_or_raise(env_name: str) -> str:
    value = os.environ.get(env_name)
    if value is None:
        raise ValueError(f"Environment variable {env_name} expected, but not set")
    return value


def get_socket_with_port() -> socket.socket:
    """A listening-ready socket bound to a free port of the loopback-or-any address (IPv4, then IPv6)."""
    last = None
    for family, addr in ((socket.AF_INET, "127.0.0.1"), (socket.AF_INET6, "::1")):
        s = socket.socket(family, socket.SOCK_STREAM)
        try:
            s.bind((addr, 0))
            s.listen(0)
            return s
        except OSError as e:
            s.close()
            last = e
    raise RuntimeError(f"Failed to create a socket: {last}")


def get_free_port() -> int:
    with contextlib.closing(get_socket_with_port()) as s:
        return s.getsockname()[1]


class macros:
    """``${local_rank}`` in the launcher's arguments is replaced by the worker's local rank."""
    local_rank = "${local_rank}"

    @staticmethod
    def substitute(args: Iterable, local_rank: str) -> List:
        return [a.replace(macros.local_rank, local_rank) if isinstance(a, str) else a for a in args]


def _seconds(timeout: Union[float, timedelta, None]) -> Optional[float]:
    if timeout is None:
        return None
    return timeout.total_seconds() if isinstance(timeout, timedelta) else float(timeout)


@contextlib.contextmanager
def store_timeout(store, timeout: Union[float, timedelta, None] = None):
    """Temporarily sets the store's operation timeout (stores without ``set_timeout`` are left alone)."""
    secs = _seconds(timeout)
    old = getattr(store, "timeout", None)
    can = secs is not None and hasattr(store, "set_timeout")
    if can:
        store.set_timeout(timedelta(seconds=secs))
    try:
        yield
    finally:
        if can and old is not None:
            store.set_timeout(old if isinstance(old, timedelta) else timedelta(seconds=float(old)))


def get_all(store, rank: int, prefix: str, world_size: int) -> List[bytes]:
    """Values of ``{prefix}{i}`` for every ``i`` (waits for each). The last reader of all ranks' check-in keys
    may clean up: every rank counts itself out under ``{prefix}/finished``."""
    data = [store.get(f"{prefix}{i}") for i in range(world_size)]
    done = store.add(f"{prefix}/finished", 1)
    if done == world_size:
        store.set(f"{prefix}/all_done", b"1")
    return data


def synchronize(store, data: bytes, rank: int, world_size: int, key_prefix: str,
                timeout: Union[float, timedelta] = 300) -> List[bytes]:
    """All-gather of one blob per rank through the store."""
    with store_timeout(store, timeout):
        store.set(f"{key_prefix}{rank}", data)
        return get_all(store, rank, key_prefix, world_size)


def barrier(store, world_size: int, key_prefix: str, barrier_timeout: Union[float, timedelta] = 300,
            rank: Optional[int] = None, rank_tracing_decoder=None, trace_timeout: float = 10) -> None:
    """Returns once ``world_size`` callers arrived. On a timeout, rank 0 names the ranks that did not arrive
    (when the callers passed their ranks)."""
    with store_timeout(store, barrier_timeout):
        if rank is not None:
            store.set(f"{key_prefix}/arrived/{rank}", b"1")
        n = store.add(f"{key_prefix}/count", 1)
        if n == world_size:
            store.set(f"{key_prefix}/last", b"1")
        try:
            store.wait([f"{key_prefix}/last"], timedelta(seconds=_seconds(barrier_timeout)))
        except Exception as e:
            if rank == 0:
                missing = [r for r in range(world_size) if not store.check([f"{key_prefix}/arrived/{r}"])]
                names = [rank_tracing_decoder(r) if rank_tracing_decoder else str(r) for r in missing]
                raise type(e)(f"barrier {key_prefix!r} timed out; ranks that did not arrive: {', '.join(names)}") from e
            raise


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
