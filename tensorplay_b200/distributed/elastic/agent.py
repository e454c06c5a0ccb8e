"""Elastic agents (worker groups, restarts): PyTorch's package of the same role; the launcher of this framework is ``distributed.run.LocalElasticAgent``."""
import importlib
import sys

sys.modules[__name__] = importlib.import_module("torch.distributed.elastic.agent")
