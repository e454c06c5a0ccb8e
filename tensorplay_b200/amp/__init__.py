"""``amp``: autocast and GradScaler (torch's policy table reproduces the reference's four cast
groups, tools/codegen/gen_autocast.py:28-131). ``GradScaler`` accepts the fused AdamW of this
package: its ``found_inf`` / ``grad_scale`` are read on the device by the kernel."""
from torch.amp import GradScaler, autocast, custom_bwd, custom_fwd, is_autocast_available  # noqa: F401
from torch.amp import autocast_mode, grad_scaler  # noqa: F401

__all__ = ["GradScaler", "autocast", "custom_bwd", "custom_fwd", "is_autocast_available"]
