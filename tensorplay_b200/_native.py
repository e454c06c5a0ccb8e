"""ctypes bindings of the in-tree native libraries.

``kernels()`` returns ``libtpb200.so`` (sm_100a CUDA kernels, C ABI) with argument types set;
``runtime()`` returns ``libtpb200rt.so`` (host runtime: store, ``.mega`` IO, symmetric memory).
On a machine with a CUDA device the kernel library is mandatory: ops raise if it is missing
instead of silently falling back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_LIBDIR = Path(__file__).resolve().parent / "_lib"
_lock = threading.Lock()
_kernels = None
_runtime = None

P = C.c_void_p
I = C.c_int
LL = C.c_longlong
F = C.c_float
U32 = C.c_uint32

_KERNEL_SIGS = {
    "tpb_gemm_bf16": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "tpb_gemm_bf16_pair": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "tpb_gemm_bf16_single": [P, P, P, P, I, I, I, I, I, I, I, I, I, I, I, F, P, P],
    "tpb_gemm_set_pair_min_tiles": [I],
    "tpb_nvtx_enable": [I],
    "tpb_nvtx_enabled": [],
    "tpb_debug_build": [],
    "tpb_debug_set_status": [P],
    "tpb_gemm_pair_resident": [],
    "tpb_gemm_pair_block_n": [I],
    "tpb_gemm_pair_trace": [P],
    "tpb_gemm_set_splitk_workspace": [P, P],
    "tpb_rmsnorm_fwd": [P, P, P, P, P, P, I, I, LL, LL, F, P],
    "tpb_rmsnorm_bwd_grid": [I, I],
    "tpb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, P, I, I, I, LL, LL, LL, P],
    "tpb_layernorm_fwd": [P, P, P, P, P, P, I, I, F, P],
    "tpb_layernorm_bwd": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, P],
    "tpb_rope": [P, P, P, P, LL, I, I, LL, LL, I, I, I, P],
    "tpb_rope_out": [P, P, P, P, P, LL, I, I, LL, LL, LL, LL, I, I, I, P],
    "tpb_swiglu_fwd": [P, P, P, LL, I, LL, P],
    "tpb_swiglu_bwd": [P, P, P, P, P, LL, I, LL, LL, P],
    "tpb_swiglu_fwd_n": [P, P, P, LL, I, LL, P, P],
    "tpb_swiglu_bwd_n": [P, P, P, P, P, LL, I, LL, LL, P, P],
    "tpb_gelu_fwd": [P, P, LL, I, P],
    "tpb_gelu_bwd": [P, P, P, LL, I, P],
    "tpb_cross_entropy": [P, P, P, P, P, LL, I, LL, LL, F, P],
    "tpb_cross_entropy_bwd": [P, P, P, P, P, P, P, LL, I, LL, LL, P],
    "tpb_flash_fwd": [P, P, P, P, P, I, I, I, I, I, I] + [LL] * 12 + [I, I, F, P, P, P, I, LL, LL],
    "tpb_flash_fwd_ex": [P, P, P, P, P, I, I, I, I, I, I] + [LL] * 12 + [I, I, F, P, P, P, I, LL, LL, I, P, P],
    "tpb_flash_bwd_ex": [P] * 10 + [I, I, I, I, I, I] + [LL] * 21 + [I, I, F, P, P, I, P, P],
    "tpb_flash_fwd_config": [I],
    "tpb_attn_split_merge": [P, P, P, P, I, I, I, I, I, LL, LL, I, LL, LL, LL, P],
    "tpb_flash_bwd": [P] * 10 + [I, I, I, I, I, I] + [LL] * 21 + [I, I, F, P, P],
    "tpb_grouped_workspace_ints": [I, I],
    "tpb_grouped_gemm": [P, P, P, P, I, I, I, I, I, I, I, I, P, P, P],
    "tpb_adamw_flat": [P, P, P, P, I, P, I, LL, F, F, F, F, F, I, F, I, P, P, P],
    "tpb_adamw_set_overlap": [I, I],
    "tpb_adamw_multi": [I, P, P, P, P, P, P, I, I, F, F, F, F, F, I, F, I, P, P, P],
    "tpb_adafactor_step": [P, P, I, P, P, P, P, P, LL, LL, F, F, F, F, F, F, F, F, P, P],
    "tpb_optim_multi": [I, I, I, P, P, P, P, P, P, P, I, F, F, F, F, F, F, P, P],
    "tpb_amp_unscale_multi": [I, P, P, I, P, P, P],
    "tpb_amp_update_scale": [P, P, P, F, F, I, P],
    "tpb_sumsq": [P, I, LL, F, P, P],
    "tpb_clip_coef": [P, F, P, P, P],
    "tpb_gemm_i8": [P, P, P, P, P, P, I, I, I, I, I, I, P, P],
    "tpb_wq_gemv": [P, P, P, P, P, P, I, I, I, I, I, LL, LL, P],
    "tpb_wq_gemv_config": [I, I],
    "tpb_lif_fwd": [P, P, P, P, I, LL, F, F, F, I, P],
    "tpb_lif_bwd": [P, P, P, P, I, LL, F, F, F, F, I, I, P],
    "tpb_quant_i8_rowwise": [P, P, P, I, I, LL, P],
    "tpb_dequant_weight": [P, P, P, P, I, I, I, I, P],
    "tpb_fp8_quant": [P, P, P, LL, I, I, I, P],
    "tpb_fp8_dequant": [P, P, P, LL, I, I, I, P],
    "tpb_embedding_fwd": [P, P, P, LL, I, LL, P],
    "tpb_embedding_bwd": [P, P, P, LL, I, LL, I, P],
    "tpb_kv_append": [P, P, P, P, I, I, I, I, I, I, I, LL, LL, LL, LL, LL, LL, P],
    "tpb_nms": [P, P, I, F, P, P, P, P],
    "tpb_roi_align_fwd": [P, P, P, I, I, I, I, I, I, I, I, F, I, I, P],
    "tpb_roi_align_bwd": [P, P, P, I, I, I, I, I, I, I, I, F, I, I, P],
    "tpb_decode_qkv_prep": [P, P, P, P, P, P, P, I, I, I, I, I, I, LL, LL, LL, LL, P],
    "tpb_sample": [P, P, P, P, I, I, LL, I, F, I, F, P],
}


class NativeUnavailable(RuntimeError):
    pass


def _load(name: str):
    path = _LIBDIR / name
    if not path.exists():
        # Build lazily when a compiler is around (developer machines, CI); the GPU boxes
        # receive the prebuilt objects with the tree.
        if os.environ.get("TPB_NO_AUTOBUILD") != "1":
            try:
                from . import _build
                _build.build_all()
            except Exception as e:  # pragma: no cover - depends on toolchain
                raise NativeUnavailable(f"{name} is not built and the in-tree build failed: {e}")
    if not path.exists():
        raise NativeUnavailable(f"{path} not found; run `python -m tensorplay_b200._build`")
    return C.CDLL(str(path), mode=C.RTLD_GLOBAL)


# kernel launches issued by one call of each entry point (for launch accounting)
_LAUNCHES = {"tpb_rmsnorm_bwd": 2, "tpb_layernorm_bwd": 3, "tpb_flash_bwd": 3, "tpb_rmsnorm_bwd_grid": 0,
             "tpb_grouped_workspace_ints": 0, "tpb_adamw_set_overlap": 0, "tpb_flash_fwd_config": 0, "tpb_gemm_set_splitk_workspace": 0, "tpb_grouped_gemm": 2}
launch_count = 0

# FLOP accounting of the native kernels: the op wrappers report every launch's floating-point work here, and an
# active ``utils.flop_counter.FlopCounterMode`` (which otherwise only sees ATen operators) adds it to its tables.
flop_sinks: list = []


def add_flops(name: str, flops: int) -> None:
    for sink in flop_sinks:
        sink(name, int(flops))



class _Counting:
    """Proxy over the ctypes library that counts kernel launches per entry point."""

    def __init__(self, lib):
        self._lib = lib
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._lib, name)
            n = _LAUNCHES.get(name, 1)

            def fn(*a, _raw=raw, _n=n):
                global launch_count
                launch_count += _n
                return _raw(*a)

            self._cache[name] = fn
        return fn


def register_sigs(lib, sigs) -> None:
    for fn, args in sigs.items():
        if hasattr(lib, fn):
            f = getattr(lib, fn)
            f.argtypes = args
            f.restype = C.c_int


def kernels():
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                debug = os.environ.get("TPB_DEBUG") == "1"
                if debug and not (_LIBDIR / "libtpb200_dbg.so").exists() and os.environ.get("TPB_NO_AUTOBUILD") != "1":
                    from . import _build
                    _build.build_kernels(debug=True)
                lib = _load("libtpb200_dbg.so" if debug else "libtpb200.so")
                register_sigs(lib, _KERNEL_SIGS)
                _kernels = _Counting(lib)
    return _kernels


def runtime():
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                _runtime = _load("libtpb200rt.so")
    return _runtime


def kernels_available() -> bool:
    try:
        kernels()
        return True
    except Exception:
        return False


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")
