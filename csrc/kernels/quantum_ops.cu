// State-vector gate application (the role of the reference's QuantumKernels.cu: one- and
// controlled one-qubit gates on a batch of complex64 state vectors).
//
// The op is a pure stream: every amplitude is read once and written once (16 bytes per complex
// pair each way), so the kernel is laid out for HBM: one thread owns the pair (i0, i0 | bit), i0
// enumerated with the target bit removed, which keeps neighbouring threads on neighbouring
// amplitudes for every target but the least significant one. Controls are a bit mask that the
// pair index must contain; pairs outside the controlled subspace are copied through.
#include <cuda_runtime.h>
#include <stdint.h>

namespace tpb {
namespace {

struct Gate2 {
  float2 m00, m01, m10, m11;
};

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}

__global__ void __launch_bounds__(256)
apply_1q_kernel(const float2* __restrict__ in, float2* __restrict__ out, long long pairs_per_state,
                long long total_pairs, int bit_pos, unsigned long long ctrl_mask, Gate2 g) {
  const unsigned long long bit = 1ull << bit_pos;
  const unsigned long long low = bit - 1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total_pairs;
       i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long b = (unsigned long long)(i / pairs_per_state);
    const unsigned long long r = (unsigned long long)(i % pairs_per_state);
    const unsigned long long i0 = ((r & ~low) << 1) | (r & low);  // insert a 0 at bit_pos
    const unsigned long long base = b * (unsigned long long)pairs_per_state * 2ull;
    const float2 a0 = in[base + i0], a1 = in[base + (i0 | bit)];
    float2 o0 = a0, o1 = a1;
    if ((i0 & ctrl_mask) == ctrl_mask) {
      const float2 p = cmul(g.m00, a0), q = cmul(g.m01, a1), s = cmul(g.m10, a0), t = cmul(g.m11, a1);
      o0 = make_float2(p.x + q.x, p.y + q.y);
      o1 = make_float2(s.x + t.x, s.y + t.y);
    }
    out[base + i0] = o0;
    out[base + (i0 | bit)] = o1;
  }
}

}  // namespace
}  // namespace tpb

extern "C" {

// state / out: [batch, 2^n_qubits] complex64 (may alias); target and controls are qubit numbers
// with qubit 0 the most significant bit; m: the 2 x 2 matrix as 8 floats (re, im, row-major).
int tpb_quantum_apply_1q(const void* state, void* out, int batch, int n_qubits, int target,
                         const int* controls, int n_controls, const float* m, void* stream) {
  if (batch <= 0 || n_qubits <= 0 || n_qubits > 40 || target < 0 || target >= n_qubits) return -1;
  unsigned long long mask = 0;
  for (int i = 0; i < n_controls; ++i) {
    if (controls[i] < 0 || controls[i] >= n_qubits || controls[i] == target) return -2;
    mask |= 1ull << (n_qubits - 1 - controls[i]);
  }
  tpb::Gate2 g;
  g.m00 = make_float2(m[0], m[1]);
  g.m01 = make_float2(m[2], m[3]);
  g.m10 = make_float2(m[4], m[5]);
  g.m11 = make_float2(m[6], m[7]);
  const long long pairs = 1ll << (n_qubits - 1);
  const long long total = pairs * batch;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  tpb::apply_1q_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float2*>(state), static_cast<float2*>(out), pairs, total, n_qubits - 1 - target, mask, g);
  return (int)cudaGetLastError();
}

}  // extern "C"
