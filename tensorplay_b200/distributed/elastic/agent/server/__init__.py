"""Agent-side servers: ``health_check_server`` (own); the agent API classes resolve to PyTorch's."""
from .health_check_server import HealthCheckServer, create_healthcheck_server

__all__ = ["HealthCheckServer", "create_healthcheck_server"]


def __getattr__(name):
    import importlib
    if name == "LocalElasticAgent":
        from ....run import LocalElasticAgent
        return LocalElasticAgent
    for mod in ("torch.distributed.elastic.agent.server", "torch.distributed.elastic.agent.server.api"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
