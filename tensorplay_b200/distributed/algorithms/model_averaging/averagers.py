"""Import path of the averager classes (tensorplay/distributed/algorithms/model_averaging/averagers.py); defined in the package."""
from . import ModelAverager, PeriodicModelAverager  # noqa: F401
