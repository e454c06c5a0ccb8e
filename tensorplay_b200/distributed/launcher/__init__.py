"""Programmatic launcher API (tensorplay/distributed/launcher/api.py): ``LaunchConfig`` +
``elastic_launch`` of the ``tprun`` agent."""
from ..run import ChildFailedError, LaunchConfig, LocalElasticAgent, elastic_launch, main  # noqa: F401

__all__ = ["ChildFailedError", "LaunchConfig", "LocalElasticAgent", "elastic_launch", "main"]
