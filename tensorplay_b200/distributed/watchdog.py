"""In-process watchdog: a thread that flags (or aborts on) steps and streams that stop making
progress, plus the host side of the device status word.

``Watchdog.heartbeat()`` is called by the training loop; if no heartbeat arrives within
``cpu_timeout`` seconds, or a recorded CUDA event does not complete within ``stream_timeout``,
the configured action runs (log / raise in the main thread at the next heartbeat / exit).
Environment: ``TP_WATCHDOG_TIMEOUT``, ``TP_WATCHDOG_ACTION`` (after
tensorplay/distributed/_watchdog.py:73-221). Failure of a peer is detected without faulting any
GPU: device waits are bounded and report through ``ops.check_status``; ranks publish heartbeats
in the store so that others can see a missing peer before their next launch."""
from __future__ import annotations

import logging
import os
import threading
import time
from typing import Callable, Optional

log = logging.getLogger("tensorplay_b200.watchdog")


class WatchdogTimeout(RuntimeError):
    pass


class Watchdog:
    def __init__(self, cpu_timeout: Optional[float] = None, stream_timeout: Optional[float] = None,
                 action: Optional[str] = None, on_timeout: Optional[Callable[[str], None]] = None,
                 poll_interval: float = 0.05):
        self.cpu_timeout = cpu_timeout if cpu_timeout is not None else float(os.environ.get("TP_WATCHDOG_TIMEOUT", "0") or 0)
        self.stream_timeout = stream_timeout
        self.action = action or os.environ.get("TP_WATCHDOG_ACTION", "log")
        self.on_timeout = on_timeout
        self.poll = poll_interval
        self._last = time.monotonic()
        self._event = None
        self._event_t = None
        self._stop = threading.Event()
        self.tripped: Optional[str] = None
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def heartbeat(self, cuda_event=None) -> None:
        if self.tripped and self.action == "raise":
            msg, self.tripped = self.tripped, None
            raise WatchdogTimeout(msg)
        self._last = time.monotonic()
        if cuda_event is not None:
            self._event, self._event_t = cuda_event, time.monotonic()

    def _trip(self, msg: str) -> None:
        if self.tripped:
            return
        self.tripped = msg
        log.error("watchdog: %s", msg)
        if self.on_timeout:
            self.on_timeout(msg)
        if self.action == "exit":
            os._exit(17)

    def _loop(self) -> None:
        while not self._stop.wait(self.poll):
            now = time.monotonic()
            if self.cpu_timeout and now - self._last > self.cpu_timeout:
                self._trip(f"no heartbeat for {now - self._last:.2f}s (limit {self.cpu_timeout}s)")
            ev = self._event
            if ev is not None and self.stream_timeout:
                try:
                    done = ev.query()
                except Exception:
                    done = True
                if done:
                    self._event = None
                elif now - self._event_t > self.stream_timeout:
                    self._trip(f"CUDA stream made no progress for {now - self._event_t:.2f}s")

    def close(self) -> None:
        self._stop.set()
        self._thread.join(timeout=1)


class PeerHeartbeat:
    """Rank liveness through the store: every rank bumps ``hb/<rank>``; ``missing()`` lists the
    ranks whose counter did not move within ``timeout`` seconds."""

    def __init__(self, store, rank: int, world: int, timeout: float = 5.0):
        self.store, self.rank, self.world, self.timeout = store, rank, world, timeout
        self._seen = {}

    def beat(self) -> None:
        self.store.add(f"hb/{self.rank}", 1)

    def missing(self):
        now = time.monotonic()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self.store.add(f"hb/{r}", 0)
            last_v, last_t = self._seen.get(r, (None, now))
            if v != last_v:
                self._seen[r] = (v, now)
            elif now - last_t > self.timeout:
                out.append(r)
        return out
