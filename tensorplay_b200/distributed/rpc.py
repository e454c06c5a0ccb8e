"""``distributed.rpc`` is not part of this framework: the reference builds it on tensorpipe for
multi-host parameter servers and remote modules (tensorplay/distributed/rpc, src/distributed/rpc),
which a single 8-GPU box with one process per GPU does not use. The module exists so that feature
probes (``rpc.is_available()``) answer instead of failing on import."""


class RPCUnavailableError(AttributeError, RuntimeError):
    """Raised on any use of the RPC surface (an ``AttributeError`` too, so ``hasattr`` probes answer False)."""


def is_available() -> bool:
    return False


def __getattr__(name):
    raise RPCUnavailableError(f"tensorplay_b200.distributed.rpc.{name}: RPC and distributed autograd are not provided "
                       "(single-box framework); use process-group collectives or the TCP store")
