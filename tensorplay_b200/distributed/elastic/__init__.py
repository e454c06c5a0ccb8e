"""Elastic training: the local agent that supervises and restarts workers lives in
``distributed.run`` (``tprun``); the dynamic rendezvous over this package's stores, the file-based
watchdog timers, the agent's health-check server, structured events, metric streams, the process contexts
with error files and log teeing, and the store helpers are implemented in the sub-packages here
(tensorplay/distributed/elastic/**)."""
from . import events, metrics, multiprocessing, utils  # noqa: F401

from ..run import ChildFailedError, LaunchConfig, LocalElasticAgent, elastic_launch  # noqa: F401
from . import agent, rendezvous, timer  # noqa: F401

__all__ = ["ChildFailedError", "LaunchConfig", "LocalElasticAgent", "elastic_launch", "events", "metrics",
           "multiprocessing", "rendezvous", "timer", "utils", "agent"]
