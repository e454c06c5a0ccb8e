"""Import path of the averaging helpers (model_averaging/utils.py in the reference); defined in the package."""
from . import average_parameters, average_parameters_or_parameter_groups, get_params_to_average  # noqa: F401
