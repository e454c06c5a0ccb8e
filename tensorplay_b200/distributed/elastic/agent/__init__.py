"""Elastic agents: the launcher of this framework is ``distributed.run.LocalElasticAgent``; the
health-check server of an agent lives in ``agent.server.health_check_server``; other names resolve
to PyTorch's package of the same role."""
from . import server  # noqa: F401


def __getattr__(name):
    import importlib
    if name == "LocalElasticAgent":
        from ...run import LocalElasticAgent
        return LocalElasticAgent
    for mod in ("torch.distributed.elastic.agent", "torch.distributed.elastic.agent.server",
                "torch.distributed.elastic.agent.server.api"):
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
