"""Import path of ``HierarchicalModelAverager`` (model_averaging/hierarchical_model_averager.py in the reference); defined in the package."""
from . import HierarchicalModelAverager  # noqa: F401
