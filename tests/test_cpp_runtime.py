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


def _tsan_works(tmp_path) -> bool:
    src = tmp_path / "probe.cpp"
    src.write_text("int main(){return 0;}\n")
    exe = tmp_path / "probe"
    r = subprocess.run(["g++", "-fsanitize=thread", str(src), "-o", str(exe)], capture_output=True)
    return r.returncode == 0 and subprocess.run([str(exe)], capture_output=True).returncode == 0


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_cpp_runtime_thread_sanitizer(tmp_path):
    """The store (server thread + clients), the reducer, the `.mega` IO and the token loader (worker threads)
    compiled with ThreadSanitizer and run through the same native unit test: no data race may be reported."""
    if not _tsan_works(tmp_path):
        pytest.skip("ThreadSanitizer runtime is not available")
    rt = ROOT / "csrc" / "runtime"
    exe = tmp_path / "test_runtime_tsan"
    srcs = [str(ROOT / "tests" / "cpp" / "test_runtime.cpp")] + [str(rt / n) for n in
                                                                ("store.cpp", "reducer.cpp", "mega_io.cpp", "token_loader.cpp")]
    cuda_inc = Path(shutil.which("nvcc")).resolve().parent.parent / "include" if shutil.which("nvcc") else Path("/usr/local/cuda/include")
    subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=thread", "-pthread", "-I", str(rt), "-I", str(cuda_inc),
                    *srcs, "-o", str(exe), "-ldl", "-lrt"], check=True)
    work = tmp_path / "work"
    work.mkdir()
    env = dict(**__import__("os").environ, TSAN_OPTIONS="halt_on_error=0 exitcode=66")
    out = subprocess.run([str(exe), str(work)], capture_output=True, text=True, timeout=600, env=env)
    assert "WARNING: ThreadSanitizer" not in out.stderr, out.stderr[-4000:]
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all runtime checks passed" in out.stdout
