"""Import path of ``noop_hook`` (ddp_comm_hooks/debugging_hooks.py in the reference)."""
from . import noop_hook  # noqa: F401
