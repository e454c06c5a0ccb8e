"""Watchdog timers between workers and their agent through a file.

A worker wraps a region in ``with expires(after=seconds):``; entering appends an *acquire* record
(pid, scope, deadline) to the timer file, leaving appends a *release*. The agent's
``FileTimerServer`` thread tails the file and, when a deadline passes without its release, signals
the worker (SIGKILL by default) - a worker stuck in a collective or a data loader is reaped instead
of hanging the job. Appends of a short line with ``O_APPEND`` are atomic, so many workers share one
file without a lock (the reference uses a named pipe,
tensorplay/distributed/elastic/timer/file_based_local_timer.py).
"""
from __future__ import annotations

import contextlib
import json
import os
import signal
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple


@dataclass
class FileTimerRequest:
    version: int
    worker_pid: int
    scope_id: str
    expiration_time: float   # < 0: release
    signal: int = int(signal.SIGKILL)

    def to_json(self) -> str:
        return json.dumps({"version": self.version, "pid": self.worker_pid, "scope_id": self.scope_id,
                           "expiration_time": self.expiration_time, "signal": self.signal})


class FileTimerClient:
    def __init__(self, file_path: str, signal=signal.SIGKILL):
        self.file_path, self.signal = file_path, int(signal)

    def _append(self, req: FileTimerRequest) -> None:
        fd = os.open(self.file_path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o600)
        try:
            os.write(fd, (req.to_json() + "\n").encode())
        finally:
            os.close(fd)

    def acquire(self, scope_id: str, expiration_time: float) -> None:
        self._append(FileTimerRequest(1, os.getpid(), scope_id, expiration_time, self.signal))

    def release(self, scope_id: str) -> None:
        self._append(FileTimerRequest(1, os.getpid(), scope_id, -1, self.signal))


class FileTimerServer:
    """Tails ``file_path`` every ``max_interval`` seconds and reaps workers whose timers expired.
    ``on_expire(pid, scope)`` (optional) is called before the signal; ``kill`` can be replaced in tests."""

    def __init__(self, file_path: str, run_id: str = "", max_interval: float = 1.0, daemon: bool = True,
                 on_expire: Optional[Callable[[int, str], None]] = None, kill: Callable[[int, int], None] = os.kill):
        self.file_path, self.run_id, self.max_interval = file_path, run_id, max_interval
        self._timers: Dict[Tuple[int, str], Tuple[float, int]] = {}
        self._pos = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=daemon)
        self._on_expire, self._kill = on_expire, kill
        self.expired: list = []
        open(file_path, "a").close()

    def start(self) -> None:
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread.is_alive():
            self._thread.join(timeout=5)

    def _read_new(self) -> None:
        with open(self.file_path, "rb") as f:
            f.seek(self._pos)
            data = f.read()
        end = data.rfind(b"\n")
        if end < 0:
            return
        self._pos += end + 1
        for line in data[: end].splitlines():
            try:
                r = json.loads(line)
            except ValueError:
                continue
            key = (int(r["pid"]), str(r["scope_id"]))
            if r["expiration_time"] < 0:
                self._timers.pop(key, None)
            else:
                self._timers[key] = (float(r["expiration_time"]), int(r.get("signal", signal.SIGKILL)))

    def run_once(self) -> None:
        self._read_new()
        now = time.time()
        for (pid, scope), (deadline, sig) in list(self._timers.items()):
            if now < deadline:
                continue
            self.expired.append((pid, scope))
            if self._on_expire is not None:
                self._on_expire(pid, scope)
            try:
                self._kill(pid, sig)
            except ProcessLookupError:
                pass
            for key in [k for k in self._timers if k[0] == pid]:
                self._timers.pop(key, None)   # the worker is gone: drop all its timers

    def _loop(self) -> None:
        while not self._stop.wait(self.max_interval):
            self.run_once()


_client: Optional[FileTimerClient] = None


def configure(client: FileTimerClient) -> None:
    """Install the process-wide client that :func:`expires` uses."""
    global _client
    _client = client


@contextlib.contextmanager
def expires(after: float, scope: Optional[str] = None, client: Optional[FileTimerClient] = None):
    """The enclosed block must finish within ``after`` seconds or the agent reaps this process."""
    c = client or _client
    if c is None:
        raise RuntimeError("no timer client configured: call configure(FileTimerClient(path)) first")
    scope_id = scope or f"scope_{threading.get_ident()}_{time.monotonic_ns()}"
    c.acquire(scope_id, time.time() + after)
    try:
        yield
    finally:
        c.release(scope_id)
