"""``backends.cuda``: PyTorch's module plus ``is_available``, ``get_name`` and ``is_ck_sdpa_available``."""
import torch as _torch
import torch.backends.cuda as _impl

globals().update({_n: getattr(_impl, _n) for _n in dir(_impl) if not _n.startswith("_")})


def is_available() -> bool:
    """Was this PyTorch built with CUDA and is a device visible?"""
    return bool(_impl.is_built() and _torch.cuda.is_available())


def get_name(device=None) -> str:
    """Name of the device (``"NVIDIA B200"``), or ``"cpu"`` without one."""
    return _torch.cuda.get_device_name(device) if _torch.cuda.is_available() else "cpu"


def is_ck_sdpa_available() -> bool:
    """The composable-kernel attention backend belongs to another vendor's stack: never on this one."""
    return False


def __getattr__(name):
    return getattr(_impl, name)
