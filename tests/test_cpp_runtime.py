"""Builds and runs the native (C++) unit test of the host runtime library."""
import shutil
import subprocess
from pathlib import Path

import pytest

from tensorplay_b200 import _native

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_cpp_runtime(tmp_path):
    _native.runtime()  # builds libtpb200rt.so if it is missing
    libdir = ROOT / "tensorplay_b200" / "_lib"
    exe = tmp_path / "test_runtime"
    subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", str(ROOT / "tests" / "cpp" / "test_runtime.cpp"),
                    f"-L{libdir}", "-ltpb200rt", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all runtime checks passed" in out.stdout
