"""Import path of the post-local-SGD hook and its state (ddp_comm_hooks/post_localSGD_hook.py in the reference)."""
from ... import algorithms as _a

PostLocalSGDState, post_localSGD_hook = _a.PostLocalSGDState, _a.post_localSGD_hook
