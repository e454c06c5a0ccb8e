"""Programmatic launcher API (tensorplay/distributed/launcher/api.py): ``LaunchConfig`` +
``elastic_launch`` of the ``tprun`` agent."""
from ..run import ChildFailedError, LaunchConfig, LocalElasticAgent, elastic_launch, main  # noqa: F401

__all__ = ["ChildFailedError", "LaunchConfig", "LocalElasticAgent", "elastic_launch", "main"]


def __getattr__(name):
    """``launch_agent`` and the launch configuration resolve to PyTorch's elastic launcher."""
    import importlib
    for mod in ['torch.distributed.launcher', 'torch.distributed.launcher.api']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
