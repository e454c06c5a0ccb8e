// Fused multi-step leaky integrate-and-fire neuron (the role of the reference's fused LIF
// operator, README "Spiking" section: one launch for all T steps, forward and BPTT).
//
//   h[t] = v[t-1] + (x[t] - (v[t-1] - v_reset)) / tau      s[t] = (h[t] >= v_th)
//   v[t] = h[t] (1 - s[t]) + v_reset s[t]                  (hard reset)
//
// The op is a stream over [T, N]: a thread owns four neighbouring neurons and walks the time axis,
// so every step is one 16-byte (fp32) or 8-byte (bf16) load and store per thread, fully coalesced
// across the warp, with the state in registers. The forward optionally writes the pre-reset
// membrane h (fp32) for the backward, which walks time in reverse with the arctan surrogate
//   ds/dh = (alpha / 2) / (1 + (pi / 2 * alpha * (h - v_th))^2).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tpb {
namespace {

struct F4 {
  float v[4];
};

template <typename T>
__device__ __forceinline__ F4 load4(const T* p);
template <>
__device__ __forceinline__ F4 load4<float>(const float* p) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  return F4{{a.x, a.y, a.z, a.w}};
}
template <>
__device__ __forceinline__ F4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 a = *reinterpret_cast<const uint2*>(p);
  return F4{{__uint_as_float(a.x << 16), __uint_as_float(a.x & 0xffff0000u), __uint_as_float(a.y << 16),
             __uint_as_float(a.y & 0xffff0000u)}};
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const F4& f);
template <>
__device__ __forceinline__ void store4<float>(float* p, const F4& f) {
  *reinterpret_cast<float4*>(p) = make_float4(f.v[0], f.v[1], f.v[2], f.v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const F4& f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f.v[0], f.v[1]), b = __floats2bfloat162_rn(f.v[2], f.v[3]);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&a);
  o.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = o;
}

template <typename T>
__global__ void __launch_bounds__(256)
lif_fwd_kernel(const T* __restrict__ x, T* __restrict__ s, float* __restrict__ h_out,
               float* __restrict__ v_io, int steps, long long n, float inv_tau, float v_th, float v_reset) {
  const long long groups = n / 4;
  for (long long gi = blockIdx.x * (long long)blockDim.x + threadIdx.x; gi < groups;
       gi += (long long)gridDim.x * blockDim.x) {
    const long long c = gi * 4;
    F4 v;
    if (v_io) v = load4<float>(v_io + c);
    else v = F4{{v_reset, v_reset, v_reset, v_reset}};
    // the next step's input is requested before this step's arithmetic
    F4 xt = load4<T>(x + c);
    for (int t = 0; t < steps; ++t) {
      F4 xn = xt;
      if (t + 1 < steps) xn = load4<T>(x + (long long)(t + 1) * n + c);
      F4 h, sp;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        h.v[i] = v.v[i] + (xt.v[i] - (v.v[i] - v_reset)) * inv_tau;
        sp.v[i] = h.v[i] >= v_th ? 1.f : 0.f;
        v.v[i] = h.v[i] >= v_th ? v_reset : h.v[i];
      }
      store4<T>(s + (long long)t * n + c, sp);
      if (h_out) store4<float>(h_out + (long long)t * n + c, h);
      xt = xn;
    }
    if (v_io) store4<float>(v_io + c, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
lif_bwd_kernel(const T* __restrict__ gs, const float* __restrict__ h, T* __restrict__ gx,
               const float* __restrict__ gv_last, int steps, long long n, float inv_tau, float v_th,
               float v_reset, float alpha, int detach_reset) {
  const long long groups = n / 4;
  const float half_alpha = 0.5f * alpha, k = 1.5707963267948966f * alpha;
  for (long long gi = blockIdx.x * (long long)blockDim.x + threadIdx.x; gi < groups;
       gi += (long long)gridDim.x * blockDim.x) {
    const long long c = gi * 4;
    F4 gv;
    if (gv_last) gv = load4<float>(gv_last + c);
    else gv = F4{{0.f, 0.f, 0.f, 0.f}};
    for (int t = steps - 1; t >= 0; --t) {
      const F4 g = load4<T>(gs + (long long)t * n + c);
      const F4 ht = load4<float>(h + (long long)t * n + c);
      F4 out;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float u = ht.v[i] - v_th;
        const float spike = u >= 0.f ? 1.f : 0.f;
        const float ku = k * u;
        const float sg = half_alpha / (1.f + ku * ku);
        float gsp = g.v[i];
        if (!detach_reset) gsp += gv.v[i] * (v_reset - ht.v[i]);
        const float gh = gv.v[i] * (1.f - spike) + gsp * sg;
        out.v[i] = gh * inv_tau;
        gv.v[i] = gh * (1.f - inv_tau);
      }
      store4<T>(gx + (long long)t * n + c, out);
    }
  }
}

inline int grid_for(long long n) {
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace
}  // namespace tpb

extern "C" {

// x, s: [steps, n] fp32 (dtype 0) or bf16 (dtype 1); n a multiple of 4; h_out (fp32 [steps, n]) and
// v_io (fp32 [n], initial membrane in, final membrane out) may be null.
int tpb_lif_fwd(const void* x, void* s, float* h_out, float* v_io, int steps, long long n, float tau,
                float v_th, float v_reset, int dtype, void* stream) {
  if (steps <= 0 || n <= 0 || (n & 3) || tau <= 0.f) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    tpb::lif_fwd_kernel<float><<<tpb::grid_for(n), 256, 0, st>>>((const float*)x, (float*)s, h_out, v_io, steps, n,
                                                               1.f / tau, v_th, v_reset);
  else if (dtype == 1)
    tpb::lif_fwd_kernel<__nv_bfloat16><<<tpb::grid_for(n), 256, 0, st>>>(
        (const __nv_bfloat16*)x, (__nv_bfloat16*)s, h_out, v_io, steps, n, 1.f / tau, v_th, v_reset);
  else
    return -2;
  return (int)cudaGetLastError();
}

int tpb_lif_bwd(const void* gs, const float* h, void* gx, const float* gv_last, int steps, long long n,
                float tau, float v_th, float v_reset, float alpha, int detach_reset, int dtype, void* stream) {
  if (steps <= 0 || n <= 0 || (n & 3) || tau <= 0.f) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    tpb::lif_bwd_kernel<float><<<tpb::grid_for(n), 256, 0, st>>>((const float*)gs, h, (float*)gx, gv_last, steps, n,
                                                               1.f / tau, v_th, v_reset, alpha, detach_reset);
  else if (dtype == 1)
    tpb::lif_bwd_kernel<__nv_bfloat16><<<tpb::grid_for(n), 256, 0, st>>>(
        (const __nv_bfloat16*)gs, h, (__nv_bfloat16*)gx, gv_last, steps, n, 1.f / tau, v_th, v_reset, alpha,
        detach_reset);
  else
    return -2;
  return (int)cudaGetLastError();
}

}  // extern "C"
