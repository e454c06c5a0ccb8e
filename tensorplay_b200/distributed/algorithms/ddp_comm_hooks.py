"""DDP communication hooks under the reference's module path
(tensorplay/distributed/algorithms/ddp_comm_hooks/{default_hooks,quantization_hooks,post_localSGD_hook,
debugging_hooks,powerSGD_hook}.py). ``allreduce_hook``, the fp16/bf16 compression hooks, ``powerSGD_hook``, the
8-bit quantisation hooks, ``post_localSGD_hook`` and ``noop_hook`` are this framework's; the remaining names
(``ddp_zero_hook``, ``mixed_precision_hooks``, ``optimizer_overlap_hooks``) resolve to PyTorch's modules, which
act on PyTorch's own DDP class."""
from torch.distributed.algorithms.ddp_comm_hooks import *  # noqa: F401,F403
from torch.distributed.algorithms.ddp_comm_hooks import powerSGD_hook as powerSGD  # noqa: F401

from . import (PostLocalSGDState, _done, allreduce_hook, bf16_compress_hook, fp16_compress_hook,  # noqa: F401
               post_localSGD_hook, powerSGD_hook, quantization_perchannel_hook, quantization_pertensor_hook)


def noop_hook(_state, bucket):
    """Returns the bucket unreduced: isolates the cost of communication when timing a step."""
    return _done(bucket.buffer())


class _Namespace:
    pass


default_hooks = _Namespace()
default_hooks.allreduce_hook, default_hooks.fp16_compress_hook = allreduce_hook, fp16_compress_hook
default_hooks.bf16_compress_hook = bf16_compress_hook
quantization_hooks = _Namespace()
quantization_hooks.quantization_pertensor_hook = quantization_pertensor_hook
quantization_hooks.quantization_perchannel_hook = quantization_perchannel_hook
post_localSGD = _Namespace()
post_localSGD.PostLocalSGDState, post_localSGD.post_localSGD_hook = PostLocalSGDState, post_localSGD_hook
debugging_hooks = _Namespace()
debugging_hooks.noop_hook = noop_hook
