// Fused Adafactor step for sm_100a: factored second moments (row and column variances) for matrices,
// a full variance for vectors, fp32 state and fp32 (master) weights, gradients in bf16 or fp32,
// optional bf16 parameter emit. Every scalar of the rule (RMS of the parameter, norm of the update,
// mean of the row variances) stays on the device: the host never waits.
//
// The rule is torch.optim.Adafactor's (and the reference's p10/include/OptimizerMTA.cuh:1522-1753):
//   beta2_t = 1 - step^decay, rho = min(lr, 1/sqrt(step)), alpha = max(eps2, rms(p)) * rho
//   p *= 1 - lr * weight_decay
//   matrices: row_var <- lerp(row_var, mean_c g^2, 1 - beta2_t); col_var likewise over rows;
//             v = row_var x col_var / max(mean(row_var), eps1^2)
//   vectors : v <- lerp(v, g^2, 1 - beta2_t)
//   u = g * rsqrt(max(v, eps1^2)); p -= alpha / max(1, rms(u) / d) * u
//
// A matrix takes four launches (statistics, moment update, norm of the update, apply); tiles of
// 64 rows x 256 columns, one column per thread, so that loads are coalesced along rows and the
// column sums stay in a register.
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int kAfRows = 64;
constexpr int kAfCols = 256;

struct AfArgs {
  float* p;
  const void* g;
  __nv_bfloat16* model;
  float* row_var;   // [R]
  float* col_var;   // [C]
  float* var;       // vectors: [n]
  // scratch: [0] sum p^2, [1] sum u^2, [2] mean(row_var), [3] unused, then row sums [R], column sums [C]
  float* scratch;
  long long R, C;
  float lr, weight_decay, eps1sq, eps2, d, omb2, rho;
  float grad_scale;
  const float* found_inf;
};

template <typename GradT>
__device__ __forceinline__ float af_grad(const void* g, long long i, float scale) {
  if constexpr (sizeof(GradT) == 2) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i]) * scale;
  else return reinterpret_cast<const float*>(g)[i] * scale;
}

__device__ __forceinline__ float block_sum_256(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 8) t = sh[threadIdx.x];
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  __syncthreads();
  return t;  // valid in thread 0
}

// ---- matrices, pass 1: row sums and column sums of g^2, sum of p^2
template <typename GradT>
__global__ void __launch_bounds__(kAfCols)
af_stats_kernel(const AfArgs a) {
  if (a.found_inf && *a.found_inf != 0.f) return;
  __shared__ float sh[8];
  __shared__ float rs[kAfRows];
  const long long c = (long long)blockIdx.x * kAfCols + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * kAfRows;
  const long long r1 = min(r0 + kAfRows, a.R);
  float* rowsum = a.scratch + 4;
  float* colsum = rowsum + a.R;
  float col = 0.f, pp = 0.f;
  const bool live = c < a.C;
  if (threadIdx.x < kAfRows) rs[threadIdx.x] = 0.f;
  __syncthreads();
  for (long long r = r0; r < r1; ++r) {
    float g2 = 0.f;
    if (live) {
      const float g = af_grad<GradT>(a.g, r * a.C + c, a.grad_scale);
      const float w = a.p[r * a.C + c];
      g2 = g * g;
      col += g2;
      pp += w * w;
    }
    // the row's share of this tile: one shared-memory add per warp, no block barrier per row
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) g2 += __shfl_xor_sync(0xffffffffu, g2, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(&rs[r - r0], g2);
  }
  __syncthreads();
  if (threadIdx.x < r1 - r0) atomicAdd(rowsum + r0 + threadIdx.x, rs[threadIdx.x]);
  if (live) atomicAdd(colsum + c, col);
  const float ps = block_sum_256(pp, sh);
  if (threadIdx.x == 0) atomicAdd(a.scratch + 0, ps);
}

// ---- matrices, pass 2 (one CTA): the two moment vectors and the mean of the row variances
__global__ void __launch_bounds__(1024)
af_moments_kernel(const AfArgs a) {
  if (a.found_inf && *a.found_inf != 0.f) return;
  __shared__ float sh[32];
  const float* rowsum = a.scratch + 4;
  const float* colsum = rowsum + a.R;
  float acc = 0.f;
  for (long long r = threadIdx.x; r < a.R; r += blockDim.x) {
    const float old = a.row_var[r];
    const float nv = old + a.omb2 * (rowsum[r] / (float)a.C - old);
    a.row_var[r] = nv;
    acc += nv;
  }
  for (long long c = threadIdx.x; c < a.C; c += blockDim.x) {
    const float old = a.col_var[c];
    a.col_var[c] = old + a.omb2 * (colsum[c] / (float)a.R - old);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = sh[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) a.scratch[2] = t / (float)a.R;
  }
}

__device__ __forceinline__ float af_update(const AfArgs& a, float g, float rv, float cv, float inv_mean) {
  const float v = fmaxf(rv * cv * inv_mean, a.eps1sq);
  return g * rsqrtf(v);
}

// ---- matrices, pass 3: sum of u^2 ; pass 4 (APPLY): the parameter update
template <typename GradT, bool APPLY>
__global__ void __launch_bounds__(kAfCols)
af_update_kernel(const AfArgs a) {
  if (a.found_inf && *a.found_inf != 0.f) return;
  __shared__ float sh[8];
  const long long c = (long long)blockIdx.x * kAfCols + threadIdx.x;
  const long long r0 = (long long)blockIdx.y * kAfRows;
  const long long r1 = min(r0 + kAfRows, a.R);
  const bool live = c < a.C;
  const float inv_mean = 1.f / fmaxf(a.scratch[2], a.eps1sq);
  const float cv = live ? a.col_var[c] : 0.f;
  float step = 0.f, keep = 1.f;
  if (APPLY) {
    const float n = (float)(a.R * a.C);
    const float alpha = fmaxf(a.eps2, sqrtf(a.scratch[0] / n)) * a.rho;
    const float denom = fmaxf(1.f, sqrtf(a.scratch[1] / n) / a.d);
    step = alpha / denom;
    keep = 1.f - a.lr * a.weight_decay;
  }
  float uu = 0.f;
  for (long long r = r0; r < r1; ++r) {
    if (!live) continue;
    const long long i = r * a.C + c;
    const float u = af_update(a, af_grad<GradT>(a.g, i, a.grad_scale), a.row_var[r], cv, inv_mean);
    if (APPLY) {
      const float w = a.p[i] * keep - step * u;
      a.p[i] = w;
      if (a.model) a.model[i] = __float2bfloat16(w);
    } else {
      uu += u * u;
    }
  }
  if (!APPLY) {
    const float t = block_sum_256(uu, sh);
    if (threadIdx.x == 0) atomicAdd(a.scratch + 1, t);
  }
}

// ---- vectors, pass 1: variance update, sum p^2, sum u^2 ; pass 2: apply
template <typename GradT, bool APPLY>
__global__ void __launch_bounds__(256)
af_vector_kernel(const AfArgs a) {
  if (a.found_inf && *a.found_inf != 0.f) return;
  __shared__ float sh[8];
  const long long n = a.C;
  float step = 0.f, keep = 1.f;
  if (APPLY) {
    const float alpha = fmaxf(a.eps2, sqrtf(a.scratch[0] / (float)n)) * a.rho;
    const float denom = fmaxf(1.f, sqrtf(a.scratch[1] / (float)n) / a.d);
    step = alpha / denom;
    keep = 1.f - a.lr * a.weight_decay;
  }
  float pp = 0.f, uu = 0.f;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float g = af_grad<GradT>(a.g, i, a.grad_scale);
    if (!APPLY) {
      const float old = a.var[i];
      const float nv = old + a.omb2 * (g * g - old);
      a.var[i] = nv;
      const float u = g * rsqrtf(fmaxf(nv, a.eps1sq));
      const float w = a.p[i];
      pp += w * w;
      uu += u * u;
    } else {
      const float u = g * rsqrtf(fmaxf(a.var[i], a.eps1sq));
      const float w = a.p[i] * keep - step * u;
      a.p[i] = w;
      if (a.model) a.model[i] = __float2bfloat16(w);
    }
  }
  if (!APPLY) {
    const float t0 = block_sum_256(pp, sh);
    const float t1 = block_sum_256(uu, sh);
    if (threadIdx.x == 0) { atomicAdd(a.scratch + 0, t0); atomicAdd(a.scratch + 1, t1); }
  }
}

}  // namespace tpb

using namespace tpb;

// Floats of scratch that tpb_adafactor_step needs for a tensor of R x C (vectors: R = 1).
extern "C" long long tpb_adafactor_scratch_floats(long long R, long long C) { return 4 + (R > 1 ? R + C : 0); }

// One Adafactor step of one tensor. R > 1: matrix [R, C] with row_var [R] and col_var [C]; R == 1: vector of C
// elements with var [C]. omb2 = step^beta2_decay, rho = min(lr, 1/sqrt(step)) are computed by the caller (host
// scalars that depend on the step count only). scratch: tpb_adafactor_scratch_floats floats, cleared here.
extern "C" int tpb_adafactor_step(float* p, const void* g, int grad_bf16, void* model, float* row_var, float* col_var,
                                  float* var, float* scratch, long long R, long long C, float lr, float weight_decay,
                                  float eps1, float eps2, float d, float omb2, float rho, float grad_scale,
                                  const float* found_inf, void* stream) {
  TPB_NVTX("tpb_adafactor_step");
  if (R <= 0 || C <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  AfArgs a;
  a.p = p; a.g = g; a.model = (__nv_bfloat16*)model; a.row_var = row_var; a.col_var = col_var; a.var = var;
  a.scratch = scratch; a.R = R; a.C = C; a.lr = lr; a.weight_decay = weight_decay; a.eps1sq = eps1 * eps1;
  a.eps2 = eps2; a.d = d; a.omb2 = omb2; a.rho = rho; a.grad_scale = grad_scale; a.found_inf = found_inf;
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)tpb_adafactor_scratch_floats(R, C) * 4, s);
  if (e != cudaSuccess) return (int)e;
  if (R > 1) {
    if (!row_var || !col_var) return -2;
    if ((C + kAfCols - 1) / kAfCols > 2147483647LL || (R + kAfRows - 1) / kAfRows > 65535) return -2;
    dim3 grid((unsigned)((C + kAfCols - 1) / kAfCols), (unsigned)((R + kAfRows - 1) / kAfRows));
    if (grad_bf16) {
      af_stats_kernel<__nv_bfloat16><<<grid, kAfCols, 0, s>>>(a);
      af_moments_kernel<<<1, 1024, 0, s>>>(a);
      af_update_kernel<__nv_bfloat16, false><<<grid, kAfCols, 0, s>>>(a);
      af_update_kernel<__nv_bfloat16, true><<<grid, kAfCols, 0, s>>>(a);
    } else {
      af_stats_kernel<float><<<grid, kAfCols, 0, s>>>(a);
      af_moments_kernel<<<1, 1024, 0, s>>>(a);
      af_update_kernel<float, false><<<grid, kAfCols, 0, s>>>(a);
      af_update_kernel<float, true><<<grid, kAfCols, 0, s>>>(a);
    }
  } else {
    if (!var) return -2;
    long long blocks = (C + 255) / 256;
    if (blocks > 1184) blocks = 1184;
    if (grad_bf16) {
      af_vector_kernel<__nv_bfloat16, false><<<(unsigned)blocks, 256, 0, s>>>(a);
      af_vector_kernel<__nv_bfloat16, true><<<(unsigned)blocks, 256, 0, s>>>(a);
    } else {
      af_vector_kernel<float, false><<<(unsigned)blocks, 256, 0, s>>>(a);
      af_vector_kernel<float, true><<<(unsigned)blocks, 256, 0, s>>>(a);
    }
  }
  return (int)cudaGetLastError();
}
