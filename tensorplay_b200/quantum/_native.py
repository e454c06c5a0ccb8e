"""CUDA path of the one-qubit (optionally controlled) gate on complex64 states."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch
from torch import Tensor

from .. import _native
from ..ops._common import lib, ptr, stream_ptr, use_native

_SIG = {"tpb_quantum_apply_1q": [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                  C.c_void_p, C.c_void_p]}
_registered = False


def apply_1q_native(state: Tensor, matrix: Tensor, target: int, controls: Tuple[int, ...]) -> Optional[Tensor]:
    """Out-of-place gate application by the stream kernel, or ``None`` when the native library or
    the layout does not fit (the caller then takes the tensor-op path)."""
    global _registered
    if not use_native(state) or not state.is_contiguous():
        return None
    raw = lib()._lib
    if not hasattr(raw, "tpb_quantum_apply_1q"):
        return None
    if not _registered:
        _native.register_sigs(raw, _SIG)
        _registered = True
    n = state.dim() - 1
    m = torch.view_as_real(matrix.detach().to(torch.complex64).cpu().contiguous()).reshape(-1).tolist()
    marr = (C.c_float * 8)(*m)
    carr = (C.c_int * max(1, len(controls)))(*controls)
    out = torch.empty_like(state)
    _native.check(lib().tpb_quantum_apply_1q(ptr(state), ptr(out), state.shape[0], n, target,
                                             C.cast(carr, C.c_void_p), len(controls),
                                             C.cast(marr, C.c_void_p), stream_ptr()), "tpb_quantum_apply_1q")
    return out


# the reference has a package at this path: deeper module names resolve to views of the pack
__path__: list = []
