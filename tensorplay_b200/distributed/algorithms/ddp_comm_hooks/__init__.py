"""DDP communication hooks under the reference's module path
(tensorplay/distributed/algorithms/ddp_comm_hooks/{default_hooks,quantization_hooks,post_localSGD_hook,
debugging_hooks,powerSGD_hook}.py). ``allreduce_hook``, the fp16/bf16 compression hooks, ``powerSGD_hook``, the
8-bit quantisation hooks, ``post_localSGD_hook`` and ``noop_hook`` are this framework's; the remaining names
(``ddp_zero_hook``, ``mixed_precision_hooks``, ``optimizer_overlap_hooks``) resolve to PyTorch's modules, which
act on PyTorch's own DDP class."""
from torch.distributed.algorithms.ddp_comm_hooks import *  # noqa: F401,F403

from .. import (PostLocalSGDState, _done, allreduce_hook, bf16_compress_hook, fp16_compress_hook,  # noqa: F401
                quantization_perchannel_hook, quantization_pertensor_hook)


def noop_hook(_state, bucket):
    """Returns the bucket unreduced: isolates the cost of communication when timing a step."""
    return _done(bucket.buffer())


# As in the reference, ``post_localSGD_hook`` and ``powerSGD_hook`` name MODULES here (the functions of the same
# names live inside them, and at ``distributed.algorithms``).
from . import debugging_hooks, default_hooks, post_localSGD_hook, powerSGD_hook, quantization_hooks  # noqa: E402,F401

post_localSGD, powerSGD = post_localSGD_hook, powerSGD_hook



def __getattr__(name):
    """``ddp_zero_hook``, ``optimizer_overlap_hooks``, ``mixed_precision_hooks``: PyTorch's modules (they act on PyTorch's DDP)."""
    if name in ("ddp_zero_hook", "optimizer_overlap_hooks", "mixed_precision_hooks"):
        import importlib
        return importlib.import_module(f"torch.distributed.algorithms.ddp_comm_hooks.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
