"""``amp``: autocast and GradScaler (torch's policy table reproduces the reference's four cast
groups, tools/codegen/gen_autocast.py:28-131). ``GradScaler`` here unscales the gradients and
updates the loss scale with this package's kernels (p10/src/backend/cuda/AmpKernels.cu:63, :95 in
the reference); the fused optimizers of ``tensorplay_b200.optim`` read ``found_inf`` /
``grad_scale`` on the device."""
from collections import defaultdict as _defaultdict

import torch as _torch
from torch.amp import GradScaler as _TorchGradScaler
from torch.amp import autocast, custom_bwd, custom_fwd, is_autocast_available  # noqa: F401
from torch.amp import autocast_mode, grad_scaler  # noqa: F401


class GradScaler(_TorchGradScaler):
    """torch's scaler with the two device-side steps on this package's kernels: the multi-tensor
    unscale + non-finite check and the scale update (no host synchronisation in either)."""

    def _unscale_grads_(self, optimizer, inv_scale, found_inf, allow_fp16):
        from ..ops.optim import amp_unscale_
        per_device = _defaultdict(list)
        with _torch.no_grad():
            for group in optimizer.param_groups:
                for p in group["params"]:
                    if p.grad is None:
                        continue
                    if (not allow_fp16) and p.grad.dtype == _torch.float16:
                        raise ValueError("Attempting to unscale FP16 gradients.")
                    g = p.grad._values() if p.grad.is_sparse else p.grad
                    per_device[g.device].append(g)
            out = {}
            for dev, grads in per_device.items():
                fi = found_inf.to(dev) if found_inf.device != dev else found_inf
                amp_unscale_(grads, inv_scale.to(dev) if inv_scale.device != dev else inv_scale, fi)
                out[dev] = fi
        return out

    def update(self, new_scale=None):
        if not self._enabled or new_scale is not None:
            return super().update(new_scale)
        from ..ops.optim import amp_update_scale_
        _scale, _growth_tracker = self._check_scale_growth_tracker("update")
        found = [fi.to(_scale.device, non_blocking=True) for state in self._per_optimizer_states.values()
                 for fi in state["found_inf_per_device"].values()]
        assert found, "No inf checks were recorded prior to update."
        combined = found[0]
        for f in found[1:]:
            combined = combined + f
        amp_update_scale_(_scale, _growth_tracker, combined, self._growth_factor, self._backoff_factor,
                          self._growth_interval)
        from torch.amp.grad_scaler import _refresh_per_optimizer_state
        self._per_optimizer_states = _defaultdict(_refresh_per_optimizer_state)


__all__ = ["GradScaler", "autocast", "custom_bwd", "custom_fwd", "is_autocast_available"]
