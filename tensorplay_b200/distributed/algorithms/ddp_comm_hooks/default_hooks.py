"""Import path of the all-reduce and compression hooks (ddp_comm_hooks/default_hooks.py in the reference)."""
from ... import algorithms as _a

allreduce_hook, fp16_compress_hook, bf16_compress_hook = _a.allreduce_hook, _a.fp16_compress_hook, _a.bf16_compress_hook
