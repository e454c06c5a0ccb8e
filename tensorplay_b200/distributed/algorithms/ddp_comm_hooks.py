"""DDP communication hooks under the reference's module path: the hooks of this framework
(``allreduce_hook``, ``fp16_compress_hook``, ``bf16_compress_hook``, ``powerSGD_hook``) plus PyTorch's hook
modules (``default_hooks``, ``powerSGD_hook`` module, ``quantization_hooks`` ...)."""
from torch.distributed.algorithms.ddp_comm_hooks import *  # noqa: F401,F403
from torch.distributed.algorithms.ddp_comm_hooks import default_hooks, powerSGD_hook as powerSGD, quantization_hooks  # noqa: F401

from . import allreduce_hook, bf16_compress_hook, fp16_compress_hook, powerSGD_hook  # noqa: F401
