"""``profiler``: torch.profiler plus NVTX range helpers and a launch counter for our kernels."""
from torch.profiler import *  # noqa: F401,F403
from torch.profiler import ProfilerActivity, profile, record_function, schedule, tensorboard_trace_handler  # noqa: F401

from .. import _native


def kernel_launches() -> int:
    """Number of launches of this package's kernels so far in the process."""
    return _native.launch_count


class nvtx_range:
    """Context manager pushing an NVTX range (visible in Nsight tools)."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        return False


class nvtx_kernels:
    """While active, every launching entry point of the kernel library pushes an NVTX range named after
    itself (``tpb_gemm_bf16``, ``tpb_flash_fwd_ex``, ...) around its host side, so a timeline attributes
    each kernel to the library call that queued it. Off otherwise: one predictable branch per call."""

    def __enter__(self):
        lib = _native.kernels()
        self._was = lib.tpb_nvtx_enabled()
        lib.tpb_nvtx_enable(1)
        return self

    def __exit__(self, *exc):
        _native.kernels().tpb_nvtx_enable(self._was)
        return False


def merge_distributed_traces(paths, out_path) -> str:
    """Merge the Chrome-trace files that the ranks of a job exported (``.json`` or ``.json.gz``) into
    one document: the events of rank ``r`` keep their order and get process ids offset by
    ``r * 10_000_000``, so the ranks show as separate process groups on one time axis. The rank is read
    from the file's ``distributedInfo.rank`` (PyTorch's profiler writes it when the process group is
    initialised), else it is the file's position in ``paths``.
    After tensorplay/profiler/_chrome_trace_export.py:379-404."""
    import gzip
    import json
    import os

    def opener(path, mode):
        path = os.fspath(path)
        return gzip.open(path, mode + "t", encoding="utf-8") if path.endswith(".gz") else open(path, mode, encoding="utf-8")
    merged = {"traceEvents": [], "displayTimeUnit": "ns", "distributedInfo": {"merged_ranks": []}}
    for i, path in enumerate(paths):
        with opener(path, "r") as f:
            doc = json.load(f)
        if isinstance(doc, list):                      # the bare-array form of the trace format
            doc = {"traceEvents": doc}
        rank = doc.get("distributedInfo", {}).get("rank")
        rank = i if rank is None else int(rank)
        merged["distributedInfo"]["merged_ranks"].append(rank)
        for event in doc.get("traceEvents", []):
            event = dict(event)
            if isinstance(event.get("pid"), int) or (isinstance(event.get("pid"), str) and event["pid"].lstrip("-").isdigit()):
                event["pid"] = rank * 10_000_000 + int(event["pid"])
            merged["traceEvents"].append(event)
    merged["traceName"] = os.fspath(out_path)
    with opener(out_path, "w") as f:
        json.dump(merged, f)
    return os.fspath(out_path)


def __getattr__(name):
    """Event containers, ``emit_nvtx`` / ``emit_itt`` and the rest of the profiler surface resolve to PyTorch's."""
    import importlib
    for mod in ['torch.profiler', 'torch.autograd.profiler', 'torch.autograd.profiler_util', 'torch.cuda.nvtx']:
        try:
            return getattr(importlib.import_module(mod), name)
        except (ImportError, AttributeError):
            continue
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

from .. import _views as _views  # noqa: E402

_views.install(__name__, max_depth=1,
               names=("_chrome_trace_export", "_schedule", "profiler_util"))
