"""Dynamic rendezvous for elastic jobs on a key-value store.

All nodes share ONE state record (JSON under a single key). A node changes it by reading the
record, applying its change and writing it back with compare-and-set: the write only lands if
nobody changed the record in between (the *fencing*: a stale writer loses and retries on the fresh
state), so joins, departures and the closing of a round are linearised without a coordinator.

A round: nodes join the participant set; when at least ``min_nodes`` are present the round waits
``last_call_s`` for late comers (or until ``max_nodes``), then it is marked complete, ranks are
assigned by sorted node name and every participant returns ``(store, rank, world_size)`` with a
store prefix unique to the round. Nodes that arrive while a round is complete go to the wait list
(``num_nodes_waiting() > 0`` tells running agents to restart into a bigger round). Every node
refreshes a keep-alive stamp; participants whose stamp is older than ``keep_alive_s *
keep_alive_max_attempts`` are evicted by whoever next touches the state, which reopens the round.

Counterpart in the reference: tensorplay/distributed/elastic/rendezvous/dynamic_rendezvous.py:215-538
(``_RendezvousState``, keep-alive, ``_DistributedRendezvousOpExecutor``).
"""
from __future__ import annotations

import itertools
import json
import os
import socket
import threading
import time
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

from ...store import PrefixStore


class RendezvousClosedError(RuntimeError):
    pass


class RendezvousTimeoutError(TimeoutError):
    pass


class RendezvousStateError(RuntimeError):
    pass


@dataclass
class RendezvousSettings:
    run_id: str
    min_nodes: int
    max_nodes: int
    join_timeout_s: float = 600.0
    last_call_s: float = 1.0
    close_timeout_s: float = 30.0
    keep_alive_s: float = 5.0
    keep_alive_max_attempts: int = 3

    def __post_init__(self):
        if not 1 <= self.min_nodes <= self.max_nodes:
            raise ValueError("need 1 <= min_nodes <= max_nodes")


def _fresh_state() -> dict:
    return {"round": 0, "complete": False, "closed": False, "deadline": None, "participants": {}, "wait_list": [],
            "last_heartbeats": {}}


class DynamicRendezvousHandler:
    def __init__(self, store, settings: RendezvousSettings, node_name: Optional[str] = None,
                 clock: Callable[[], float] = time.time):
        self.store, self.settings = store, settings
        self.node = node_name or f"{socket.gethostname()}_{os.getpid()}_{id(self) & 0xffff}"
        self._key = f"rdzv/{settings.run_id}/state"
        self._clock = clock
        self._stop = threading.Event()
        self._beat: Optional[threading.Thread] = None
        self._write_seq = itertools.count(1)   # shared by the caller's thread and the heartbeat thread

    # ---- fenced state updates
    def _read(self) -> Tuple[dict, bytes]:
        raw = self.store.get(self._key) if self.store.check([self._key]) else b""
        return (json.loads(raw) if raw else _fresh_state()), raw

    def _update(self, fn: Callable[[dict], Optional[dict]]) -> dict:
        """Apply ``fn`` to the shared record until the compare-and-set wins; ``fn`` returns the new
        record, or None to leave it unchanged. Every written record carries a tag that is unique to the
        writer and the attempt: two writers that derive the same new record from the same old one would
        otherwise both read their own bytes back from the compare-and-set and both count it as won."""
        for _ in range(10000):
            state, raw = self._read()
            state.pop("_w", None)
            base = json.dumps(state, sort_keys=True)
            self._evict_dead(state)
            new = fn(state)
            if new is None:
                return state
            new.pop("_w", None)
            if json.dumps(new, sort_keys=True) == base:
                return new
            tagged = dict(new)
            tagged["_w"] = f"{self.node}#{id(self)}#{next(self._write_seq)}"
            blob = json.dumps(tagged, sort_keys=True).encode()
            got = self.store.compare_set(self._key, raw, blob)
            if got == blob:
                return new
            time.sleep(0.001)
        raise RendezvousStateError("could not update the rendezvous state (too much contention)")

    def _evict_dead(self, state: dict) -> None:
        ttl = self.settings.keep_alive_s * self.settings.keep_alive_max_attempts
        now = self._clock()
        dead = [n for n, t in state["last_heartbeats"].items() if now - t > ttl and n != self.node]
        for n in dead:
            state["last_heartbeats"].pop(n, None)
            if n in state["participants"]:
                state["participants"].pop(n)
                # a member of a finished round died: the round is void, survivors re-rendezvous
                if state["complete"]:
                    state["complete"] = False
                    state["round"] += 1
                    state["participants"] = {}
                    state["deadline"] = None
            if n in state["wait_list"]:
                state["wait_list"].remove(n)

    # ---- keep-alive
    def _start_heartbeat(self) -> None:
        if self._beat is not None:
            return

        def loop():
            while not self._stop.wait(self.settings.keep_alive_s):
                try:
                    self._update(self._stamp)
                except Exception:
                    pass
        self._beat = threading.Thread(target=loop, daemon=True)
        self._beat.start()

    def _stamp(self, state: dict) -> dict:
        state["last_heartbeats"][self.node] = self._clock()
        return state

    # ---- API
    def next_rendezvous(self):
        """Blocks until this node is part of a complete round; returns ``(store, rank, world_size)``."""
        s = self.settings
        t_end = time.time() + s.join_timeout_s
        self._start_heartbeat()

        def join(state: dict) -> dict:
            if state["closed"]:
                raise RendezvousClosedError(f"rendezvous {s.run_id!r} is closed")
            state["last_heartbeats"][self.node] = self._clock()
            if state["complete"]:
                if self.node in state["participants"]:
                    return state
                if self.node not in state["wait_list"]:
                    state["wait_list"].append(self.node)
                return state
            if self.node in state["wait_list"]:
                state["wait_list"].remove(self.node)
            if self.node not in state["participants"] and len(state["participants"]) < s.max_nodes:
                state["participants"][self.node] = 0
            n = len(state["participants"])
            if n >= s.min_nodes and state["deadline"] is None:
                state["deadline"] = self._clock() + s.last_call_s
            if n >= s.max_nodes or (state["deadline"] is not None and self._clock() >= state["deadline"] and n >= s.min_nodes):
                for rank, name in enumerate(sorted(state["participants"])):
                    state["participants"][name] = rank
                state["complete"] = True
                state["deadline"] = None
                # nodes that waited during the previous round start the next one themselves
            return state

        joined_round = None
        while True:
            state = self._update(join)
            if state["complete"] and self.node in state["participants"]:
                rank, world = state["participants"][self.node], len(state["participants"])
                store = PrefixStore(f"rdzv/{s.run_id}/round{state['round']}", self.store)
                return store, rank, world
            if state["complete"] and self.node in state["wait_list"]:
                # a finished round is running without us: it restarts when its agents see the wait list
                pass
            if time.time() > t_end:
                self._update(self._leave)
                raise RendezvousTimeoutError(f"rendezvous {s.run_id!r}: no complete round within {s.join_timeout_s} s")
            time.sleep(0.02)
            _ = joined_round

    def _leave(self, state: dict) -> dict:
        state["participants"].pop(self.node, None)
        if self.node in state["wait_list"]:
            state["wait_list"].remove(self.node)
        state["last_heartbeats"].pop(self.node, None)
        return state

    def restart_round(self) -> None:
        """Void the current round (an agent saw waiting nodes or lost a worker): everybody,
        waiting nodes included, joins the next one."""
        def fn(state: dict) -> Optional[dict]:
            if not state["complete"]:
                return None
            state["complete"] = False
            state["round"] += 1
            state["participants"] = {}
            state["deadline"] = None
            return state
        self._update(fn)

    def num_nodes_waiting(self) -> int:
        return len(self._read()[0]["wait_list"])

    def is_closed(self) -> bool:
        return bool(self._read()[0]["closed"])

    def set_closed(self) -> None:
        def fn(state: dict) -> dict:
            state["closed"] = True
            return state
        self._update(fn)

    def get_run_id(self) -> str:
        return self.settings.run_id

    def get_backend(self) -> str:
        return "tpb-dynamic"

    def shutdown(self) -> bool:
        self._stop.set()
        try:
            self._update(self._leave)
            return True
        except Exception:
            return False


def create_handler(store, run_id: str, min_nodes: int, max_nodes: int, **kw) -> DynamicRendezvousHandler:
    return DynamicRendezvousHandler(store, RendezvousSettings(run_id, min_nodes, max_nodes, **kw))
