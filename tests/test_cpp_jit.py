"""JIT loading of C++ kernels (CPU path; the CUDA path is compiled, not run, without a GPU)."""
import shutil

import pytest
import torch

from tensorplay_b200.utils import comparison, cpp_jit

CPP = r'''
extern "C" int axpy_f32(float* y, const float* x, long long n, double a) {
  for (long long i = 0; i < n; ++i) y[i] += (float)a * x[i];
  return 0;
}
extern "C" int fails(long long code) { return (int)code; }
'''

CU = r'''
__global__ void scale_kernel(float* x, long long n, float a) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i < n) x[i] *= a;
}
extern "C" int scale_f32(float* x, long long n, double a, void* stream) {
  scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, (float)a);
  return (int)cudaGetLastError();
}
'''


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_load_inline_cpp_and_cache(tmp_path):
    mod = cpp_jit.load_inline("axpy", cpp_sources=CPP, functions={"axpy_f32": None}, build_directory=str(tmp_path))
    x, y = torch.arange(8, dtype=torch.float32), torch.ones(8)
    assert mod.axpy_f32(y, x, 8, 0.5) == 0
    assert comparison.allclose(y, 1 + 0.5 * torch.arange(8.0))
    assert mod.fails(7) == 7
    with pytest.raises(AttributeError):
        mod.not_exported
    # same sources: the cached artefact is reused; AOT path + load_module give the same functions
    path = cpp_jit.build_inline("axpy", cpp_sources=CPP, build_directory=str(tmp_path))
    assert path == mod.path and len(list(tmp_path.glob("*.so"))) == 1
    again = cpp_jit.load_module(path)
    assert again.axpy_f32(y, x, 8, 1.0) == 0 and float(y[7]) == 1 + 1.5 * 7
    with pytest.raises(RuntimeError):
        cpp_jit.build_inline("broken", cpp_sources="this is not C++", build_directory=str(tmp_path))


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc")
def test_build_inline_cuda_for_sm100a(tmp_path):
    path = cpp_jit.build_inline("scale", cuda_sources=CU, build_directory=str(tmp_path))
    assert path.endswith(".so")
