"""tensorplay_b200: a Blackwell-native deep-learning framework with the public API of TensorPlay.

The framework layer is PyTorch (``Tensor`` is ``torch.Tensor``, autograd is torch's); the hot
ops are hand-written sm_100a kernels (``tensorplay_b200.ops``), the parallel runtime
(``tensorplay_b200.parallel`` and ``tensorplay_b200.distributed``) is built on NVLink peer memory
with NCCL kept for point-to-point and as the baseline, and a plain-PyTorch CPU path is the
correctness oracle. Top-level names follow tensorplay/__init__.py:270-760 of the reference: what
coincides with torch semantics is re-exported, what the reference adds lives in this package.

``import tensorplay_b200 as tp`` (or ``tensorplay_b200.compat.install_alias()`` to make
``import tensorplay`` resolve here).
"""
from __future__ import annotations

import importlib as _importlib
import sys as _sys

import torch as _torch

__version__ = "0.1.0"

# ---- everything torch exposes at top level (functions, dtypes, grad modes, ...)
import types as _types

for _n in dir(_torch):
    if _n.startswith("_"):
        continue
    _v = getattr(_torch, _n)
    if isinstance(_v, _types.ModuleType):
        continue  # sub-packages are resolved below (ours first, torch's lazily)
    globals()[_n] = _v
del _n, _v

Tensor = _torch.Tensor
DType = _torch.dtype
Device = _torch.device
dtype = _torch.dtype
device = _torch.device

# ---- own subpackages (imported eagerly: they are light) and torch-backed ones (lazy)
ops = _importlib.import_module(__name__ + ".ops")
nn = _importlib.import_module(__name__ + ".nn")
optim = _importlib.import_module(__name__ + ".optim")
amp = _importlib.import_module(__name__ + ".amp")
serialization = _importlib.import_module(__name__ + ".serialization")
from .serialization import inspect_checkpoint, load, save  # noqa: E402
from .nn.generation import sample  # noqa: E402

_LAZY_OWN = {"distributed", "utils", "models", "parallel", "cuda", "profiler", "autograd", "compat",
             "multiprocessing", "testing", "quantization", "metrics", "snn", "library", "quantum", "lumen", "vision", "linalg", "sparse", "func", "audio", "config", "ao", "backends"}
_LAZY_TORCH = {"fft", "special", "distributions", "futures", "hub", "onnx", "mps",
               "masked", "nested", "monitor", "accelerator", "export", "fx", "random",
               "signal", "overrides", "package", "storage", "types", "jit", "_numpy"}


_FALLBACK = ("export", "graph", "accelerator", "mps", "monitor", "package")


class _TorchAliasFinder:
    """Import fallback for the thin packages: ``tensorplay_b200.<pkg>.<module>`` that is not a file of
    this framework resolves to ``torch.<pkg>.<module>`` (e.g. ``optim.adam``, ``autograd.function``,
    ``profiler.profiler``, ``multiprocessing.reductions``), so module paths of the reference that only
    name PyTorch-equivalent code keep importing. Sits last on ``sys.meta_path``: own modules win."""

    _PKGS = ("optim", "autograd", "profiler", "multiprocessing", "utils", "cuda", "amp", "testing", "nn", "distributed", "ao", "backends")

    def find_spec(self, fullname, path=None, target=None):
        parts = fullname.split(".")
        if len(parts) < 2 or parts[0] != __name__:
            return None
        import importlib.util
        if len(parts) == 2 and parts[1] in _FALLBACK:
            return importlib.util.spec_from_loader(fullname, _FallbackLoader(parts[1]))
        if parts[1] in ("vision", "audio"):       # sub-modules without a file here: torchvision / torchaudio
            torch_name = ".".join(["torchvision" if parts[1] == "vision" else "torchaudio"] + parts[2:])
        elif parts[1] == "_transforms":
            torch_name = ".".join(["torch.func"] + parts[2:])
        elif parts[1] == "graph":            # the reference's name of the graph IR package
            torch_name = ".".join(["torch.fx"] + parts[2:])
        elif parts[1] in _LAZY_TORCH or (len(parts) >= 3 and parts[1] in self._PKGS):
            # whole packages that are PyTorch's (``linalg``, ``func``, ``fx`` ...), or a module path below
            # a thin package of this framework
            torch_name = "torch." + ".".join(parts[1:])
        else:
            return None
        if torch_name not in _sys.modules:        # (a loaded module may have no __spec__: torch.backends)
            try:
                if importlib.util.find_spec(torch_name) is None:
                    return None
            except (ImportError, ValueError, AttributeError):
                return None
        return importlib.util.spec_from_loader(fullname, _TorchAliasLoader(torch_name))


class _FallbackLoader:
    def __init__(self, short):
        self.short = short

    def create_module(self, spec):
        return _sys.modules.get(spec.name) or _build_fallback(self.short)

    def exec_module(self, module):
        pass


class _TorchAliasLoader:
    def __init__(self, torch_name):
        self.torch_name = torch_name

    def create_module(self, spec):
        return _importlib.import_module(self.torch_name)

    def exec_module(self, module):
        pass


class _AliasedParentFinder:
    """First on ``sys.meta_path``: a sub-module of a name that already resolved to a PyTorch (or torchvision /
    torchaudio) package must resolve to the SAME module object as its PyTorch spelling. Without this the path
    finder would follow the aliased package's ``__path__`` and execute PyTorch's source file a second time under
    the new name: duplicate classes, and operator registrations that fail the second time."""

    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        parent_name, _, tail = fullname.rpartition(".")
        parent = _sys.modules.get(parent_name)
        base = getattr(parent, "__dict__", {}).get("__wrapped_base__") if parent is not None else None
        real = getattr(base if base is not None else parent, "__name__", "")
        if parent is None or real == parent_name or real.split(".")[0] not in ("torch", "torchvision", "torchaudio"):
            return None
        import importlib.util
        target_name = f"{real}.{tail}"
        try:
            if target_name not in _sys.modules and importlib.util.find_spec(target_name) is None:
                return None
        except (ImportError, ValueError, AttributeError):
            return None
        return importlib.util.spec_from_loader(fullname, _TorchAliasLoader(target_name))


import sys as _sys  # noqa: E402

if not [f for f in _sys.meta_path if type(f).__name__ == "_TorchAliasFinder"]:
    # after the standard finders (own files win), before the view finders of the packs that were imported while
    # this module was still executing (PyTorch's module of the same path wins over a view)
    _views_at = [i for i, f in enumerate(_sys.meta_path) if type(f).__name__ == "_ViewFinder"]
    _sys.meta_path.insert(_views_at[0] if _views_at else len(_sys.meta_path), _TorchAliasFinder())
if not [f for f in _sys.meta_path if type(f).__name__ == "_AliasedParentFinder"]:
    _sys.meta_path.insert(0, _AliasedParentFinder())


def _build_fallback(name):
    """``export``, ``graph``, ``accelerator``, ``mps``, ``monitor``, ``package``, ``backends``: PyTorch's packages with
    the reference's extra top-level names looked up in PyTorch's sub-modules."""
    from . import _fallback
    full = f"{__name__}.{name}"
    if name == "export":
        return _fallback.make(full, "torch.export", search=(
            "torch.export.graph_signature", "torch.export.dynamic_shapes", "torch.export.exported_program",
            "torch.export.pt2_archive._package", "torch.export.pt2_archive", "torch.export.unflatten"),
            extra={"export_for_training": getattr(_torch.export, "export_for_training", _torch.export.export),
                   "GraphSignature": _torch.export.graph_signature.ExportGraphSignature})
    if name == "graph":
        return _fallback.make(full, "torch.fx", search=(
            "torch.fx.tensor_type", "torch.fx.annotate", "torch.fx.subgraph_rewriter", "torch.fx.immutable_collections",
            "torch.fx.experimental.refinement_types", "torch.fx.experimental.graph_gradual_typechecker",
            "torchvision.models.feature_extraction", "torch.jit", "torch._higher_order_ops.while_loop",
            "torch._higher_order_ops"),
            extra={"GraphCaptureError": RuntimeError})
    if name == "accelerator":
        import contextlib
        return _fallback.make(full, "torch.accelerator", search=("torch.cuda", "torch.cuda.graphs", "torch.cuda.random"),
                              extra={"Graph": _torch.cuda.CUDAGraph, "graphs": _torch.cuda.graphs, "random": _torch.cuda.random,
                                     "empty_host_cache": getattr(_torch._C, "_host_emptyCache", lambda: None)})
    if name == "mps":
        return _fallback.make(full, "torch.mps", extra={"current_device": lambda: 0,
                                                        "memory_allocated": _torch.mps.current_allocated_memory,
                                                        "memory_reserved": _torch.mps.driver_allocated_memory})
    if name == "monitor":
        import collections
        return _fallback.make(full, "torch.monitor", extra={"StatResult": collections.namedtuple(
            "StatResult", ["name", "aggregation", "value", "count"])})
    if name == "package":
        import enum
        return _fallback.make(full, "torch.package", search=("torch.package.package_exporter",), extra={
            "PackagingErrorReason": getattr(importlib_import("torch.package.package_exporter"), "PackagingErrorReason", enum.Enum)})
    raise AttributeError(name)


def importlib_import(name):
    return _importlib.import_module(name)


def __getattr__(name):
    if name in _FALLBACK:
        mod = _sys.modules.get(f"{__name__}.{name}") or _build_fallback(name)
        globals()[name] = mod
        return mod
    if name in _LAZY_OWN:
        mod = _importlib.import_module(f"{__name__}.{name}")
        globals()[name] = mod
        return mod
    if name in _LAZY_TORCH:
        mod = _importlib.import_module(f"torch.{name}")
        globals()[name] = mod
        return mod
    if name == "graph":
        return _importlib.import_module("torch.fx")
    if name == "_transforms":   # vmap / grad / jvp / vjp transforms (tensorplay/_transforms)
        return _importlib.import_module("torch.func")
    if name in ("stax", "_stax", "primitives"):
        raise AttributeError(f"tensorplay_b200.{name}: the tracing compiler and its primitive IR are not part of this "
                             "framework (hand-written kernels instead); see tensorplay_b200.compile for CUDA-graph capture")
    return getattr(_torch, name)


def compile(model=None, *, backend: str = "cuda_graph", **kwargs):
    """``tensorplay.compile`` counterpart. There is no tracing compiler here by design: the hot
    path is hand-written kernels. ``backend="cuda_graph"`` returns a callable that captures the
    module's forward into a CUDA graph for static shapes (launch-bound inner loops);
    ``backend="eager"`` returns the module unchanged."""
    def wrap(m):
        if backend == "eager" or not _torch.cuda.is_available():
            return m
        from .cuda.graphs import make_graphed_callable
        return make_graphed_callable(m)
    return wrap if model is None else wrap(model)


def is_native_available() -> bool:
    """True when the sm_100a kernel library is built and loadable."""
    from . import _native
    return _native.kernels_available()


# ---- remaining top-level names of the reference that PyTorch spells differently
import enum as _enum  # noqa: E402
import numbers as _numbers  # noqa: E402

Scalar = _numbers.Number
MemoryFormat = _torch.memory_format
Layout = _torch.layout
bcomplex32 = _torch.complex32          # the reference's name for half-precision complex
quint1x8 = getattr(_torch, "quint2x4", _torch.quint8)   # no 1-bit quantised dtype in PyTorch: closest sub-byte type
index = _torch.index_select


class DeviceType(_enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    META = "meta"


class QScheme(_enum.Enum):
    PER_TENSOR_AFFINE = _torch.per_tensor_affine
    PER_CHANNEL_AFFINE = _torch.per_channel_affine
    PER_TENSOR_SYMMETRIC = _torch.per_tensor_symmetric
    PER_CHANNEL_SYMMETRIC = _torch.per_channel_symmetric


class DeviceMismatchError(RuntimeError):
    """Operands of one operation live on different devices."""


def get_thread_num() -> int:
    """Index of the calling thread inside an intra-op parallel region (0 outside one)."""
    return 0


def in_parallel_region() -> bool:
    return False


def get_parallel_info() -> str:
    return _torch.__config__.parallel_info()


def fork_rng(devices=None, enabled: bool = True):
    """Context manager: RNG states of the CPU and of ``devices`` are restored on exit."""
    return _torch.random.fork_rng(devices=devices, enabled=enabled)


def thread_safe_generator(seed: int = None, device="cpu"):
    """A generator of its own (not the global one), seeded explicitly or from the global stream."""
    g = _torch.Generator(device=device)
    import builtins
    g.manual_seed(builtins.int(_torch.randint(0, 2 ** 62, ()).item()) if seed is None else builtins.int(seed))
    return g


def getArtifactLogger(name: str, artifact: str):
    import logging
    return logging.getLogger(f"{name}.__{artifact}")
