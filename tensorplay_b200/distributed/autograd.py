"""``distributed.autograd`` (RPC-based distributed autograd) is not part of this framework; see
``distributed.rpc``."""
from .rpc import RPCUnavailableError


def is_available() -> bool:
    return False


def __getattr__(name):
    raise RPCUnavailableError(f"tensorplay_b200.distributed.autograd.{name}: distributed autograd rides on RPC, which is not provided")
