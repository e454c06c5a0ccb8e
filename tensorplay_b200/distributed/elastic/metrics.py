"""Metrics of the elastic agent: named groups of streams with pluggable handlers
(tensorplay/distributed/elastic/metrics/api.py: ``MetricHandler`` :59, ``MetricStream`` :89, ``configure`` :128,
``put_metric`` :172, ``prof`` :185). A metric goes to the handler configured for its group, else to the default
handler (which drops it until ``configure`` sets one).
"""
from __future__ import annotations

import abc
import functools
import time
from dataclasses import dataclass
from typing import Dict, Optional


@dataclass
class MetricData:
    timestamp: float
    group_name: str
    name: str
    value: float


class MetricsConfig:
    def __init__(self, params: Optional[Dict[str, str]] = None):
        self.params = params or {}


class MetricHandler(abc.ABC):
    @abc.abstractmethod
    def emit(self, metric_data: MetricData) -> None: ...


class ConsoleMetricHandler(MetricHandler):
    def emit(self, metric_data: MetricData) -> None:
        print(f"[{metric_data.timestamp}][{metric_data.group_name}]: {metric_data.name}={metric_data.value}")


class NullMetricHandler(MetricHandler):
    def emit(self, metric_data: MetricData) -> None:
        pass


class MetricStream:
    def __init__(self, group_name: str, handler: MetricHandler):
        self.group_name, self.handler = group_name, handler

    def add_value(self, metric_name: str, metric_value: float) -> None:
        self.handler.emit(MetricData(time.time(), self.group_name, metric_name, metric_value))


_handlers: Dict[str, MetricHandler] = {}
_default_handler: MetricHandler = NullMetricHandler()


def configure(handler: MetricHandler, group: Optional[str] = None) -> None:
    """``group=None`` sets the handler of every group without one of its own."""
    global _default_handler
    if group is None:
        _default_handler = handler
    else:
        _handlers[group] = handler


def initialize_metrics(cfg: Optional[MetricsConfig] = None) -> None:
    """Hook for deployments that configure handlers from ``cfg``; the default set-up needs nothing."""


def getStream(group: str) -> MetricStream:
    return MetricStream(group, _handlers.get(group, _default_handler))


def put_metric(metric_name: str, metric_value: float, metric_group: str = "tensorplay_elastic") -> None:
    getStream(metric_group).add_value(metric_name, metric_value)


def publish_metric(metric_group: str, metric_name: str, metric_value: float) -> None:
    put_metric(metric_name, metric_value, metric_group)


def get_elapsed_time_ms(start_time_in_seconds: float) -> int:
    return int((time.time() - start_time_in_seconds) * 1000)


def _metric_prefix(fn) -> str:
    qual = fn.__qualname__.split(".")
    return fn.__name__ if len(qual) == 1 else f"{qual[-2].lower()}.{fn.__name__}"


def prof(fn=None, group: str = "tensorplay_elastic"):
    """Decorator: publishes ``<class>.<function>.success`` or ``.failure`` (value 1) and ``.duration.ms`` per call.
    Usable bare (``@prof``) or with a group (``@prof(group="agent")``)."""
    def wrap(f):
        @functools.wraps(f)
        def wrapper(*args, **kwargs):
            key = _metric_prefix(f)
            start = time.time()
            try:
                out = f(*args, **kwargs)
                put_metric(f"{key}.success", 1, group)
                return out
            except BaseException:
                put_metric(f"{key}.failure", 1, group)
                raise
            finally:
                put_metric(f"{key}.duration.ms", get_elapsed_time_ms(start), group)
        return wrapper
    return wrap(fn) if fn is not None else wrap


def profile(group=None):
    """Older spelling of :func:`prof` with the group as the only argument."""
    return prof(group=group or "tensorplay_elastic")


# the reference has a package at this path: sub-module names without a file here resolve to PyTorch's
__path__: list = []
