"""Elastic training: the local agent that supervises and restarts workers lives in
``distributed.run`` (``tprun``); events, metrics, timers and the rendezvous registry are torch's
(tensorplay/distributed/elastic/**)."""
from torch.distributed.elastic import events, metrics, multiprocessing, rendezvous, timer, utils  # noqa: F401

from ..run import ChildFailedError, LaunchConfig, LocalElasticAgent, elastic_launch  # noqa: F401

__all__ = ["ChildFailedError", "LaunchConfig", "LocalElasticAgent", "elastic_launch", "events", "metrics",
           "multiprocessing", "rendezvous", "timer", "utils"]
