"""Key-value stores for rendezvous: ``TCPStore`` (native C++ server/client in ``libtpb200rt``),
``FileStore``, ``HashStore`` and ``PrefixStore``.

All of them subclass ``torch.distributed.Store`` so that they can be handed to
``init_process_group(store=...)``; the method set follows the reference's Python protocol
(tensorplay/distributed/_store.py:27-173: ``set/get/add/compare_set/wait/has/delete_key``).
"""
from __future__ import annotations

import ctypes as C
import fcntl
import json
import os
import threading
import time
from datetime import timedelta
from typing import Iterable, List, Optional, Union

import torch.distributed as dist

from .. import _native


class StoreTimeoutError(TimeoutError):
    pass


def _ms(timeout) -> int:
    if timeout is None:
        return -1
    if isinstance(timeout, timedelta):
        return int(timeout.total_seconds() * 1000)
    return int(float(timeout) * 1000)


def _b(v: Union[str, bytes]) -> bytes:
    return v.encode() if isinstance(v, str) else bytes(v)


def _rt():
    lib = _native.runtime()
    if not getattr(lib, "_store_sigs", False):
        lib.tpb_store_server_start.argtypes = [C.c_int, C.POINTER(C.c_int)]
        lib.tpb_store_server_start.restype = C.c_void_p
        lib.tpb_store_server_stop.argtypes = [C.c_void_p]
        lib.tpb_store_connect.argtypes = [C.c_char_p, C.c_int, C.c_int]
        lib.tpb_store_connect.restype = C.c_void_p
        lib.tpb_store_close.argtypes = [C.c_void_p]
        lib.tpb_store_set.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_char_p, C.c_longlong]
        lib.tpb_store_get.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_longlong, C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_longlong)]
        lib.tpb_store_add.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_longlong, C.POINTER(C.c_longlong)]
        lib.tpb_store_cas.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_char_p, C.c_longlong, C.c_char_p,
                                      C.c_longlong, C.POINTER(C.c_void_p), C.POINTER(C.c_longlong)]
        lib.tpb_store_wait.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.c_int, C.c_longlong]
        lib.tpb_store_check.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int), C.c_int]
        lib.tpb_store_delete.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        lib.tpb_store_num_keys.argtypes = [C.c_void_p]
        lib.tpb_store_num_keys.restype = C.c_longlong
        lib.tpb_free.argtypes = [C.c_void_p]
        lib._store_sigs = True
    return lib


class _StoreBase(dist.Store):
    """Shared conveniences on top of the primitive operations."""

    def __init__(self, timeout=timedelta(seconds=300)):
        super().__init__()
        self._timeout = timeout if isinstance(timeout, timedelta) else timedelta(seconds=float(timeout))

    # torch's Store API names
    def set_timeout(self, timeout) -> None:
        self._timeout = timeout if isinstance(timeout, timedelta) else timedelta(seconds=float(timeout))

    @property
    def timeout(self):
        return self._timeout

    def has(self, key) -> bool:
        return self.check([key])

    def compare_and_swap(self, key, expected, desired):
        return self.compare_set(key, expected, desired)

    def multi_get(self, keys):
        return [self.get(k) for k in keys]

    def multi_set(self, keys, values):
        for k, v in zip(keys, values):
            self.set(k, v)


class TCPStore(_StoreBase):
    """Client of (and, with ``is_master=True``, host of) the native TCP store."""

    def __init__(self, host_name: str = "127.0.0.1", port: int = 0, world_size: Optional[int] = None,
                 is_master: bool = False, timeout=timedelta(seconds=300), wait_for_workers: bool = False):
        super().__init__(timeout)
        self._lib = _rt()
        self._server = None
        self.host = host_name
        if is_master:
            p = C.c_int(0)
            self._server = self._lib.tpb_store_server_start(int(port), C.byref(p))
            if not self._server:
                raise OSError(f"TCPStore: cannot listen on port {port}")
            port = p.value
        self.port = int(port)
        self._client = self._lib.tpb_store_connect(_b(host_name), self.port, _ms(self._timeout))
        if not self._client:
            raise StoreTimeoutError(f"TCPStore: cannot connect to {host_name}:{self.port}")
        self.world_size = world_size
        if world_size is not None and wait_for_workers:
            n = self.add("__tpb_store_workers__", 1)
            deadline = time.time() + self._timeout.total_seconds()
            while n < world_size:
                if time.time() > deadline:
                    raise StoreTimeoutError("TCPStore: timed out waiting for workers")
                time.sleep(0.01)
                n = self.add("__tpb_store_workers__", 0)

    def set(self, key, value) -> None:
        k, v = _b(key), _b(value)
        if self._lib.tpb_store_set(self._client, k, len(k), v, len(v)) != 0:
            raise ConnectionError("TCPStore.set failed")

    def get(self, key, timeout=None) -> bytes:
        k = _b(key)
        out, n = C.c_void_p(), C.c_longlong()
        st = self._lib.tpb_store_get(self._client, k, len(k), _ms(timeout if timeout is not None else self._timeout),
                                     C.byref(out), C.byref(n))
        if st == 1:
            raise StoreTimeoutError(f"TCPStore.get({key!r}) timed out")
        if st != 0:
            raise ConnectionError("TCPStore.get failed")
        try:
            return C.string_at(out, n.value)
        finally:
            self._lib.tpb_free(out)

    def add(self, key, amount: int) -> int:
        k = _b(key)
        r = C.c_longlong()
        if self._lib.tpb_store_add(self._client, k, len(k), int(amount), C.byref(r)) != 0:
            raise ConnectionError("TCPStore.add failed")
        return r.value

    def compare_set(self, key, expected, desired) -> bytes:
        k, e, d = _b(key), _b(expected), _b(desired)
        out, n = C.c_void_p(), C.c_longlong()
        if self._lib.tpb_store_cas(self._client, k, len(k), e, len(e), d, len(d), C.byref(out), C.byref(n)) != 0:
            raise ConnectionError("TCPStore.compare_set failed")
        try:
            return C.string_at(out, n.value)
        finally:
            self._lib.tpb_free(out)

    def _pack(self, keys: Iterable):
        ks = [_b(k) for k in keys]
        lens = (C.c_int * len(ks))(*[len(k) for k in ks])
        return b"".join(ks), lens, len(ks)

    def wait(self, keys, timeout=None) -> None:
        blob, lens, n = self._pack(keys)
        st = self._lib.tpb_store_wait(self._client, blob, lens, n, _ms(timeout if timeout is not None else self._timeout))
        if st == 1:
            raise StoreTimeoutError(f"TCPStore.wait({list(keys)!r}) timed out")
        if st != 0:
            raise ConnectionError("TCPStore.wait failed")

    def check(self, keys) -> bool:
        blob, lens, n = self._pack(keys)
        return self._lib.tpb_store_check(self._client, blob, lens, n) == 0

    def delete_key(self, key) -> bool:
        k = _b(key)
        return self._lib.tpb_store_delete(self._client, k, len(k)) == 0

    def num_keys(self) -> int:
        return int(self._lib.tpb_store_num_keys(self._client))

    def close(self) -> None:
        if self._client:
            self._lib.tpb_store_close(self._client)
            self._client = None
        if self._server:
            self._lib.tpb_store_server_stop(self._server)
            self._server = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class HashStore(_StoreBase):
    """In-process store (threads of one process)."""

    def __init__(self, timeout=timedelta(seconds=300)):
        super().__init__(timeout)
        self._kv = {}
        self._cv = threading.Condition()

    def set(self, key, value) -> None:
        with self._cv:
            self._kv[_b(key)] = _b(value)
            self._cv.notify_all()

    def get(self, key, timeout=None) -> bytes:
        self.wait([key], timeout)
        return self._kv[_b(key)]

    def add(self, key, amount: int) -> int:
        with self._cv:
            v = int(self._kv.get(_b(key), b"0")) + int(amount)
            self._kv[_b(key)] = str(v).encode()
            self._cv.notify_all()
            return v

    def compare_set(self, key, expected, desired) -> bytes:
        k, e, d = _b(key), _b(expected), _b(desired)
        with self._cv:
            cur = self._kv.get(k)
            if cur is None:
                if not e:
                    self._kv[k] = d
                    self._cv.notify_all()
                    return d
                return e
            if cur == e:
                self._kv[k] = d
                self._cv.notify_all()
                return d
            return cur

    def wait(self, keys, timeout=None) -> None:
        ks = [_b(k) for k in keys]
        t = (timeout if timeout is not None else self._timeout)
        secs = t.total_seconds() if isinstance(t, timedelta) else float(t)
        with self._cv:
            if not self._cv.wait_for(lambda: all(k in self._kv for k in ks), secs):
                raise StoreTimeoutError(f"HashStore.wait({keys!r}) timed out")

    def check(self, keys) -> bool:
        return all(_b(k) in self._kv for k in keys)

    def delete_key(self, key) -> bool:
        with self._cv:
            return self._kv.pop(_b(key), None) is not None

    def num_keys(self) -> int:
        return len(self._kv)


class FileStore(_StoreBase):
    """Store backed by one JSON file guarded by ``flock`` (ranks on a shared filesystem)."""

    def __init__(self, file_name: str, world_size: int = -1, timeout=timedelta(seconds=300)):
        super().__init__(timeout)
        self.path = os.fspath(file_name)
        self.world_size = world_size
        if not os.path.exists(self.path):
            with open(self.path, "a"):
                pass

    def _txn(self, fn):
        with open(self.path, "r+") as f:
            fcntl.flock(f, fcntl.LOCK_EX)
            try:
                raw = f.read()
                kv = json.loads(raw) if raw else {}
                res, dirty = fn(kv)
                if dirty:
                    f.seek(0)
                    f.truncate()
                    f.write(json.dumps(kv))
                    f.flush()
                return res
            finally:
                fcntl.flock(f, fcntl.LOCK_UN)

    def set(self, key, value) -> None:
        k, v = _b(key).hex(), _b(value).hex()
        self._txn(lambda kv: (kv.__setitem__(k, v), True))

    def get(self, key, timeout=None) -> bytes:
        self.wait([key], timeout)
        return bytes.fromhex(self._txn(lambda kv: (kv[_b(key).hex()], False)))

    def add(self, key, amount: int) -> int:
        k = _b(key).hex()

        def fn(kv):
            v = int(bytes.fromhex(kv.get(k, b"0".hex())) or b"0") + int(amount)
            kv[k] = str(v).encode().hex()
            return v, True
        return self._txn(fn)

    def compare_set(self, key, expected, desired) -> bytes:
        k, e, d = _b(key).hex(), _b(expected), _b(desired)

        def fn(kv):
            cur = kv.get(k)
            if cur is None:
                if not e:
                    kv[k] = d.hex()
                    return d, True
                return e, False
            if bytes.fromhex(cur) == e:
                kv[k] = d.hex()
                return d, True
            return bytes.fromhex(cur), False
        return self._txn(fn)

    def wait(self, keys, timeout=None) -> None:
        t = (timeout if timeout is not None else self._timeout)
        secs = t.total_seconds() if isinstance(t, timedelta) else float(t)
        deadline = time.time() + secs
        while not self.check(keys):
            if time.time() > deadline:
                raise StoreTimeoutError(f"FileStore.wait({keys!r}) timed out")
            time.sleep(0.01)

    def check(self, keys) -> bool:
        ks = [_b(k).hex() for k in keys]
        return self._txn(lambda kv: (all(k in kv for k in ks), False))

    def delete_key(self, key) -> bool:
        k = _b(key).hex()
        return self._txn(lambda kv: (kv.pop(k, None) is not None, True))

    def num_keys(self) -> int:
        return self._txn(lambda kv: (len(kv), False))


class PrefixStore(_StoreBase):
    """Namespaces every key of an underlying store."""

    def __init__(self, prefix: str, store):
        super().__init__(getattr(store, "timeout", timedelta(seconds=300)))
        self.prefix = prefix
        self.store = store

    def _k(self, key):
        return _b(self.prefix) + b"/" + _b(key)

    def set(self, key, value): self.store.set(self._k(key), value)
    def get(self, key, timeout=None):
        return self.store.get(self._k(key), timeout) if timeout is not None else self.store.get(self._k(key))
    def add(self, key, amount): return self.store.add(self._k(key), amount)
    def compare_set(self, key, expected, desired): return self.store.compare_set(self._k(key), expected, desired)
    def wait(self, keys, timeout=None):
        ks = [self._k(k) for k in keys]
        return self.store.wait(ks, timeout) if timeout is not None else self.store.wait(ks)
    def check(self, keys): return self.store.check([self._k(k) for k in keys])
    def delete_key(self, key): return self.store.delete_key(self._k(key))
    def num_keys(self): return self.store.num_keys()
