"""Shared helpers of the op wrappers: native-library access, stream handle, device status word."""
from __future__ import annotations

import torch

from .. import _native


def use_native(*tensors: torch.Tensor) -> bool:
    """True when the op must run on the sm_100a kernels (CUDA tensors).

    A CUDA tensor never falls back to PyTorch: if the kernel library cannot be loaded the
    call raises, so that a silent library fallback cannot pass for the native path.
    """
    if not tensors or not all(t is None or t.is_cuda for t in tensors):
        return False
    _native.kernels()  # raises NativeUnavailable with a clear message
    return True


def lib():
    return _native.kernels()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return None if t is None else t.data_ptr()


_status = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device uint32 word that kernels with bounded waits write an error code into."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    w = _status.get(key)
    if w is None:
        w = torch.zeros(4, dtype=torch.int32, device=dev)
        _status[key] = w
        L = lib()
        if L.tpb_debug_build():
            # debug build: failed index checks report to the same word (site << 8 | 4)
            with torch.cuda.device(dev):
                _native.check(L.tpb_debug_set_status(w.data_ptr()), "tpb_debug_set_status")
    return w


class DeviceIndexError(IndexError):
    """Debug build only (``TPB_DEBUG=1``): a kernel's index guard found an out-of-range index."""


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (mbarrier or peer flag) ran out of time."""


def check_status(device=None, reset: bool = True) -> None:
    """Read the status word (synchronises the device) and raise if a kernel reported a time-out."""
    w = status_word(device)
    v = int(w[0].item()) & 0xFFFFFFFF
    if v:
        if reset:
            w.zero_()
        code, where = v & 0xFF, v >> 8
        if code == 4:
            raise DeviceIndexError(f"device kernel skipped an out-of-range index at check site {where}")
        names = {1: "mbarrier wait time-out", 2: "flag wait time-out", 3: "bad arguments"}
        raise DeviceWaitTimeout(f"device kernel reported {names.get(code, code)} at site {where}")


def as_2d(x: torch.Tensor):
    shape = x.shape
    return x.reshape(-1, shape[-1]), shape
