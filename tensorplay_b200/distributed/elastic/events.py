"""Structured events of the elastic agent and the rendezvous: one JSON document per event, written to a
destination chosen by name (tensorplay/distributed/elastic/events/api.py: ``Event`` :40, ``RdzvEvent`` :134;
events/__init__.py: ``record`` :44, ``record_rdzv_event`` :50, ``construct_and_record_rdzv_event`` :59).

Destinations: ``"null"`` (dropped), ``"console"`` (stderr), ``"file"`` (appends to the path in
``TPB_EVENTS_FILE``); ``register_destination`` adds more.
"""
from __future__ import annotations

import json
import logging
import os
import socket
import sys
import time
import traceback
from dataclasses import asdict, dataclass, field
from enum import Enum
from typing import Callable, Dict, Optional, Union

EventMetadataValue = Union[str, int, float, bool, None]


class EventSource(str, Enum):
    AGENT = "AGENT"
    WORKER = "WORKER"


class NodeState(str, Enum):
    INIT = "INIT"
    RUNNING = "RUNNING"
    SUCCEEDED = "SUCCEEDED"
    FAILED = "FAILED"


def _now_ms() -> int:
    return int(time.time() * 1000)


@dataclass
class Event:
    name: str
    source: EventSource
    timestamp: int = 0
    metadata: Dict[str, EventMetadataValue] = field(default_factory=dict)

    def __post_init__(self):
        if not self.timestamp:
            self.timestamp = _now_ms()

    def serialize(self) -> str:
        d = asdict(self)
        d["source"] = EventSource(self.source).value
        return json.dumps(d)

    @staticmethod
    def deserialize(data: Union[str, "Event"]) -> "Event":
        if isinstance(data, Event):
            return data
        d = json.loads(data)
        d["source"] = EventSource[d["source"]]
        return Event(**d)

    def __str__(self) -> str:
        return self.serialize()


@dataclass
class RdzvEvent:
    name: str
    run_id: str
    message: str
    hostname: str = ""
    pid: int = 0
    node_state: NodeState = NodeState.INIT
    master_endpoint: str = ""
    rank: Optional[int] = None
    local_id: Optional[int] = None
    error_trace: str = ""
    timestamp: int = 0

    def __post_init__(self):
        if not self.timestamp:
            self.timestamp = _now_ms()

    def serialize(self) -> str:
        d = asdict(self)
        d["node_state"] = NodeState(self.node_state).value
        return json.dumps(d)

    @staticmethod
    def deserialize(data: Union[str, "RdzvEvent"]) -> "RdzvEvent":
        if isinstance(data, RdzvEvent):
            return data
        d = json.loads(data)
        d["node_state"] = NodeState[d["node_state"]]
        return RdzvEvent(**d)

    def __str__(self) -> str:
        return self.serialize()


def _file_handler() -> logging.Handler:
    path = os.environ.get("TPB_EVENTS_FILE")
    return logging.FileHandler(path) if path else logging.NullHandler()


_destinations: Dict[str, Callable[[], logging.Handler]] = {
    "null": logging.NullHandler,
    "console": lambda: logging.StreamHandler(sys.stderr),
    "file": _file_handler,
}
_loggers: Dict[str, logging.Logger] = {}


def register_destination(name: str, make_handler: Callable[[], logging.Handler]) -> None:
    _destinations[name] = make_handler
    _loggers.pop(name, None)


def get_logging_handler(destination: str = "null") -> logging.Handler:
    return _destinations[destination]()


def _logger(destination: str) -> logging.Logger:
    lg = _loggers.get(destination)
    if lg is None:
        lg = logging.getLogger(f"tensorplay-elastic-events-{destination}")
        lg.setLevel(logging.INFO)
        lg.propagate = False
        for h in list(lg.handlers):
            lg.removeHandler(h)
        lg.addHandler(get_logging_handler(destination))
        _loggers[destination] = lg
    return lg


def record(event: Event, destination: str = "null") -> None:
    _logger(destination).info(event.serialize())


def record_rdzv_event(event: RdzvEvent) -> None:
    _logger(os.environ.get("TPB_RDZV_EVENTS_DESTINATION", "null")).info(event.serialize())


def construct_and_record_rdzv_event(run_id: str, message: str, node_state: NodeState, name: str = "",
                                    hostname: str = "", pid: Optional[int] = None, master_endpoint: str = "",
                                    local_id: Optional[int] = None, rank: Optional[int] = None) -> None:
    """Builds the event from where it is called (name of the calling function, this host and process, the
    active exception's traceback for a failure) and records it; nothing is built when the destination drops it."""
    if os.environ.get("TPB_RDZV_EVENTS_DESTINATION", "null") == "null":
        return
    if not name:
        name = sys._getframe(1).f_code.co_name
    trace = traceback.format_exc() if node_state == NodeState.FAILED and sys.exc_info()[0] is not None else ""
    record_rdzv_event(RdzvEvent(name=name, run_id=run_id, message=message, hostname=hostname or socket.getfqdn(),
                                pid=pid or os.getpid(), node_state=node_state, master_endpoint=master_endpoint,
                                rank=rank, local_id=local_id, error_trace=trace))


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
