"""Rendezvous URL handlers: ``env://``, ``tcp://host:port`` and ``file://path`` produce
``(store, rank, world_size)`` backed by this package's stores (the native TCP store for env/tcp),
after tensorplay/distributed/rendezvous.py:27-56, 118-277. ``init_process_group`` below feeds the
result to torch.distributed so that NCCL / gloo groups bootstrap through our store."""
from __future__ import annotations

import os
from datetime import timedelta
from typing import Callable, Dict, Iterator, Optional, Tuple
from urllib.parse import parse_qs, urlparse

import torch.distributed as dist

from .store import FileStore, PrefixStore, TCPStore

_handlers: Dict[str, Callable] = {}


def register_rendezvous_handler(scheme: str, handler: Callable) -> None:
    if scheme in _handlers:
        raise RuntimeError(f"rendezvous handler for {scheme}:// already registered")
    _handlers[scheme] = handler


def _q(url):
    return {k: v[0] for k, v in parse_qs(urlparse(url).query).items()}


def _env_handler(url: str, rank: int, world_size: int, timeout):
    q = _q(url)
    rank = int(q.get("rank", os.environ.get("RANK", rank)))
    world_size = int(q.get("world_size", os.environ.get("WORLD_SIZE", world_size)))
    addr = os.environ.get("TP_STORE_ADDR") or os.environ["MASTER_ADDR"]
    if "TP_STORE_PORT" in os.environ:  # started under tprun: reuse the agent's store
        store = TCPStore(addr, int(os.environ["TP_STORE_PORT"]), world_size, False, timeout)
        store = PrefixStore(f"gen{os.environ.get('TP_RESTART_COUNT', '0')}", store)
    else:
        store = TCPStore(addr, int(os.environ["MASTER_PORT"]), world_size, rank == 0, timeout)
    return store, rank, world_size


def _tcp_handler(url: str, rank: int, world_size: int, timeout):
    u = urlparse(url)
    q = _q(url)
    rank = int(q.get("rank", rank))
    world_size = int(q.get("world_size", world_size))
    return TCPStore(u.hostname, u.port, world_size, rank == 0, timeout), rank, world_size


def _file_handler(url: str, rank: int, world_size: int, timeout):
    u = urlparse(url)
    q = _q(url)
    rank = int(q.get("rank", rank))
    world_size = int(q.get("world_size", world_size))
    return FileStore(u.path, world_size, timeout), rank, world_size


register_rendezvous_handler("env", _env_handler)
register_rendezvous_handler("tcp", _tcp_handler)
register_rendezvous_handler("file", _file_handler)


def rendezvous(url: str = "env://", rank: int = -1, world_size: int = -1,
               timeout=timedelta(seconds=300)) -> Tuple[object, int, int]:
    scheme = urlparse(url).scheme or "env"
    if scheme not in _handlers:
        raise RuntimeError(f"no rendezvous handler for {scheme}://")
    return _handlers[scheme](url, rank, world_size, timeout)


def init_process_group(backend: str = "nccl", init_method: str = "env://", rank: int = -1, world_size: int = -1,
                       timeout=timedelta(seconds=300), **kw):
    """``torch.distributed.init_process_group`` bootstrapped through this package's store."""
    store, rank, world_size = rendezvous(init_method, rank, world_size, timeout)
    dist.init_process_group(backend, store=store, rank=rank, world_size=world_size, timeout=timeout, **kw)
    return store
