"""In-tree build of the native libraries.

``libtpb200.so``  - sm_100a CUDA kernels (``csrc/kernels/*.cu``), plain C ABI, no torch dependency.
``libtpb200rt.so`` - host runtime in C++ (``csrc/runtime/*.cpp``): TCP key-value store, ``.mega``
                    checkpoint reader/writer, symmetric-memory allocator.

Both are compiled with ``nvcc``/``g++`` straight into ``tensorplay_b200/_lib`` so that the
shared objects travel with the source tree. Objects are rebuilt only when a source or header
is newer than the object.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wno-unused-function",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-fopenmp"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _newer(src_deps, out: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in src_deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}\n{r.stdout}\n{r.stderr}")
    return r.stdout + r.stderr


def build_kernels(verbose: bool = False, ptxas_info: bool = False, debug: bool = False) -> Path:
    """``debug=True`` builds ``libtpb200_dbg.so`` with ``-DTPB_KERNEL_DEBUG``: index guards that only skip
    an access in the release build also report their site to the status word (``TPB_DEBUG=1`` loads it)."""
    src_dir = CSRC / "kernels"
    headers = list(src_dir.glob("*.cuh")) + list(src_dir.glob("*.h"))
    sources = sorted(src_dir.glob("*.cu"))
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    objs, jobs = [], []
    for s in sources:
        o = OBJDIR / (s.stem + ("_dbg.o" if debug else ".o"))
        objs.append(o)
        if _newer([s, *headers], o) or ptxas_info:
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-DTPB_KERNEL_DEBUG"] if debug else []), "-I", src_dir, "-c", s, "-o", o]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    log = []
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda c: _run(c, verbose), jobs):
                log.append(out)
    lib = LIBDIR / ("libtpb200_dbg.so" if debug else "libtpb200.so")
    if jobs or _newer(objs, lib):
        # The CUDA runtime is linked dynamically so that the library shares the runtime state
        # (per-thread current device, primary context, error state) of the process that loads
        # it - torch's autograd threads select their device through that same runtime.
        _run([_nvcc(), "-shared", "-cudart", "shared", "-o", lib, *objs, "-gencode",
              "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose)
    if ptxas_info:
        print("\n".join(log))
    return lib


def build_runtime(verbose: bool = False) -> Path:
    src_dir = CSRC / "runtime"
    sources = sorted(src_dir.glob("*.cpp"))
    headers = list(src_dir.glob("*.h"))
    OBJDIR.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    lib = LIBDIR / "libtpb200rt.so"
    if not sources:
        return lib
    cuda_inc = _cuda_home() / "include"
    objs, jobs = [], []
    for s in sources:
        o = OBJDIR / ("rt_" + s.stem + ".o")
        objs.append(o)
        if _newer([s, *headers], o):
            jobs.append(["g++", *CXX_FLAGS, "-I", src_dir, "-I", cuda_inc, "-c", s, "-o", o])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or _newer(objs, lib):
        _run(["g++", "-shared", "-o", lib, *objs, "-pthread", "-fopenmp", "-ldl", "-lrt"], verbose)
    return lib


def build_all(verbose: bool = False) -> None:
    build_kernels(verbose)
    build_runtime(verbose)


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        build_kernels(True, ptxas_info=True)
    else:
        build_all(v)
    print("built:", *sorted(p.name for p in LIBDIR.glob("*.so")))
