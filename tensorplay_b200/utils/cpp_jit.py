"""Just-in-time loading of C++ / CUDA kernels behind a plain C ABI (the role of
tensorplay/utils/cpp_jit.py: ``load_inline`` / ``load`` / ``build_inline`` / ``build`` /
``load_module``).

Sources are compiled once per content hash into a shared library (``nvcc -gencode
arch=compute_100a,code=sm_100a`` for ``.cu`` sources, ``g++`` otherwise) and loaded with ctypes. The
exported functions are ``extern "C"``; a tensor argument crosses the boundary as its data pointer
(the kernel gets shapes and strides as explicit integer arguments, like this framework's own
kernels), Python ints and floats as ``long long`` / ``double`` unless ``argtypes`` says otherwise, and
``stream=True`` appends the current CUDA stream as the last ``void*`` argument.

    mod = load_inline("scale", cuda_sources=SRC, functions={"scale_f32": None})
    mod.scale_f32(x, x.numel(), 2.0, stream=True)
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import shutil
import subprocess
from pathlib import Path
from typing import Dict, Optional, Sequence, Union

import torch

_CACHE = Path(os.environ.get("TPB_JIT_CACHE", Path.home() / ".cache" / "tensorplay_b200_jit"))
CUDA_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


class JitModule:
    """Loaded shared library; attribute access returns a callable that converts its arguments."""

    def __init__(self, path: Union[str, Path], functions: Optional[Dict[str, Optional[Sequence]]] = None):
        self.path = str(path)
        self._lib = C.CDLL(self.path)
        self._sigs = dict(functions or {})

    def __getattr__(self, name: str):
        raw = getattr(self._lib, name)          # AttributeError when the symbol is not exported
        argtypes = self._sigs.get(name)
        if argtypes is not None:
            raw.argtypes = list(argtypes)
        raw.restype = C.c_int

        def call(*args, stream: bool = False):
            conv = []
            for a in args:
                if isinstance(a, torch.Tensor):
                    conv.append(C.c_void_p(a.data_ptr()))
                elif isinstance(a, bool):
                    conv.append(C.c_int(int(a)))
                elif isinstance(a, int):
                    conv.append(C.c_longlong(a))
                elif isinstance(a, float):
                    conv.append(C.c_double(a))
                elif a is None:
                    conv.append(C.c_void_p(None))
                else:
                    conv.append(a)
            if stream:
                conv.append(C.c_void_p(torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else None))
            return raw(*conv)
        call.__name__ = name
        return call


def _compile(name: str, sources: Dict[str, str], out: Path, extra_cflags, extra_cuda_cflags, extra_ldflags,
             extra_include_paths, verbose: bool) -> None:
    out.parent.mkdir(parents=True, exist_ok=True)
    work = out.parent / (out.stem + "_src")
    work.mkdir(exist_ok=True)
    files = []
    for fname, text in sources.items():
        p = work / fname
        p.write_text(text)
        files.append(p)
    inc = [f"-I{p}" for p in (extra_include_paths or [])]
    has_cuda = any(str(f).endswith(".cu") for f in files)
    if has_cuda:
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        cmd = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-O3", "-std=c++17", "-lineinfo", *CUDA_ARCH_FLAGS,
               *(extra_cuda_cflags or []), *inc, *map(str, files), "-o", str(out), *(extra_ldflags or [])]
    else:
        cmd = ["g++", "-shared", "-fPIC", "-O2", "-std=c++17", *(extra_cflags or []), *inc, *map(str, files),
               "-o", str(out), *(extra_ldflags or [])]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(" ".join(cmd))
        print(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compilation of {name} failed:\n{r.stderr[-4000:]}")


def _key(name, sources, flags) -> str:
    h = hashlib.sha256(name.encode())
    for k in sorted(sources):
        h.update(k.encode())
        h.update(sources[k].encode())
    h.update(repr(flags).encode())
    return h.hexdigest()[:16]


def build_inline(name: str, cpp_sources: Union[str, Sequence[str], None] = None,
                 cuda_sources: Union[str, Sequence[str], None] = None, extra_cflags=None, extra_cuda_cflags=None,
                 extra_ldflags=None, extra_include_paths=None, build_directory: Optional[str] = None,
                 verbose: bool = False) -> str:
    """Compile string sources into ``<build_directory>/<name>_<hash>.so`` (cached) and return its path."""
    as_list = lambda s: [] if s is None else ([s] if isinstance(s, str) else list(s))  # noqa: E731
    sources = {f"{name}_{i}.cpp": t for i, t in enumerate(as_list(cpp_sources))}
    sources.update({f"{name}_{i}.cu": t for i, t in enumerate(as_list(cuda_sources))})
    if not sources:
        raise ValueError("no sources given")
    flags = (extra_cflags, extra_cuda_cflags, extra_ldflags, extra_include_paths)
    out = Path(build_directory or _CACHE) / f"{name}_{_key(name, sources, flags)}.so"
    if not out.exists():
        _compile(name, sources, out, extra_cflags, extra_cuda_cflags, extra_ldflags, extra_include_paths, verbose)
    return str(out)


def build(name: str, sources: Sequence[str], **kw) -> str:
    """Like :func:`build_inline` for source files on disk."""
    cpp = [Path(s).read_text() for s in sources if not str(s).endswith(".cu")]
    cu = [Path(s).read_text() for s in sources if str(s).endswith(".cu")]
    return build_inline(name, cpp or None, cu or None, **kw)


def load_module(path: str, functions: Optional[Dict[str, Optional[Sequence]]] = None) -> JitModule:
    return JitModule(path, functions)


def load_inline(name: str, cpp_sources=None, cuda_sources=None, functions: Optional[Dict[str, Optional[Sequence]]] = None,
                **kw) -> JitModule:
    """Compile (or reuse the cached build of) the sources and load them. ``functions`` maps exported
    names to ctypes argument lists (``None``: convert from the Python values at each call)."""
    return JitModule(build_inline(name, cpp_sources, cuda_sources, **kw), functions)


def load(name: str, sources: Sequence[str], functions: Optional[Dict[str, Optional[Sequence]]] = None, **kw) -> JitModule:
    return JitModule(build(name, sources, **kw), functions)
