// Fused AdamW for sm_100a: flat (one contiguous shard) and multi-tensor forms, fp32 moments and
// fp32 master weights with a bf16 (or fp32) model copy written in the same pass, optional AMP
// grad-scale / found-inf handling, global grad-norm partials and clipping coefficient read
// from device memory so that no host sync is needed.
//
// Counterpart in the reference: p10/include/OptimizerMTA.cuh:560-748 (adam_math / adam_kernel)
// and p10/src/backend/cuda/AmpKernels.cu:63-95.
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_c1, bias_c2;  // 1 - beta1^t, 1 - beta2^t
  float grad_scale;        // multiply grads by this (e.g. 1/world, 1/loss_scale)
  int maximize;
};

__device__ __forceinline__ void adamw_one(float& p, float& m, float& v, float g,
                                          const AdamHyper& h) {
  if (h.maximize) g = -g;
  p *= (1.f - h.lr * h.weight_decay);
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  float denom = sqrtf(v) / sqrtf(h.bias_c2) + h.eps;
  p -= (h.lr / h.bias_c1) * (m / denom);
}

// clip_coef (device, optional): grads are additionally multiplied by *clip_coef.
// found_inf (device, optional): if *found_inf != 0 the step is skipped.
template <typename GradT, typename ModelT>
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  const GradT* __restrict__ grad, ModelT* __restrict__ model, long long n,
                  AdamHyper h, const float* __restrict__ clip_coef,
                  const float* __restrict__ found_inf) {
  if (found_inf && *found_inf != 0.f) return;
  const float gs = h.grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long nvec = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float g[4];
    if constexpr (sizeof(GradT) == 2) {
      uint2 raw = reinterpret_cast<const uint2*>(grad)[i];
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
      float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      float4 g4 = reinterpret_cast<const float4*>(grad)[i];
      g[0] = g4.x; g[1] = g4.y; g[2] = g4.z; g[3] = g4.w;
    }
    float pp[4] = {p4.x, p4.y, p4.z, p4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) adamw_one(pp[j], mm[j], vv[j], g[j] * gs, h);
    reinterpret_cast<float4*>(master)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (model) {
      if constexpr (sizeof(ModelT) == 2) {
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(pp[0], pp[1]);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(pp[2], pp[3]);
        reinterpret_cast<uint2*>(model)[i] = o;
      } else {
        reinterpret_cast<float4*>(model)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
      }
    }
  }
  // tail (n not a multiple of 4)
  long long t0 = nvec * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t0 < n) {
    float p = master[t0], mm = m[t0], vv = v[t0];
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[t0]);
    else g = grad[t0];
    adamw_one(p, mm, vv, g * gs, h);
    master[t0] = p; m[t0] = mm; v[t0] = vv;
    if (model) {
      if constexpr (sizeof(ModelT) == 2) model[t0] = __float2bfloat16(p);
      else model[t0] = p;
    }
  }
}

// ---- multi-tensor form: up to kMtaTensors tensors and kMtaBlocks (tensor, chunk) pairs per launch
constexpr int kMtaTensors = 48;
constexpr int kMtaBlocks = 640;
constexpr int kMtaChunk = 65536;
struct MtaArgs {
  void* master[kMtaTensors];
  void* m[kMtaTensors];
  void* v[kMtaTensors];
  const void* grad[kMtaTensors];
  void* model[kMtaTensors];
  long long numel[kMtaTensors];
  unsigned char block_tensor[kMtaBlocks];
  int block_chunk[kMtaBlocks];
};

template <typename GradT, typename ModelT>
__global__ void __launch_bounds__(512)
adamw_mta_kernel(const __grid_constant__ MtaArgs a, AdamHyper h,
                 const float* __restrict__ clip_coef, const float* __restrict__ found_inf) {
  if (found_inf && *found_inf != 0.f) return;
  const float gs = h.grad_scale * (clip_coef ? *clip_coef : 1.f);
  const int t = a.block_tensor[blockIdx.x];
  const long long start = (long long)a.block_chunk[blockIdx.x] * kMtaChunk;
  const long long n = a.numel[t];
  const long long end = start + kMtaChunk < n ? start + kMtaChunk : n;
  float* master = reinterpret_cast<float*>(a.master[t]);
  float* m = reinterpret_cast<float*>(a.m[t]);
  float* v = reinterpret_cast<float*>(a.v[t]);
  const GradT* grad = reinterpret_cast<const GradT*>(a.grad[t]);
  ModelT* model = reinterpret_cast<ModelT*>(a.model[t]);
  for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
    float p = master[i], mm = m[i], vv = v[i];
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[i]);
    else g = grad[i];
    adamw_one(p, mm, vv, g * gs, h);
    master[i] = p; m[i] = mm; v[i] = vv;
    if (model) {
      if constexpr (sizeof(ModelT) == 2) model[i] = __float2bfloat16(p);
      else model[i] = p;
    }
  }
}

// Sum of squares of a flat buffer, atomically added (scaled) into *out.
template <typename T>
__global__ void __launch_bounds__(256)
sumsq_kernel(const T* __restrict__ x, long long n, float scale, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 2) f = __bfloat162float(x[i]);
    else f = x[i];
    f *= scale;
    s += f * f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float sm[8];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += sm[i];
    atomicAdd(out, t);
  }
}

// coef = min(1, max_norm / (sqrt(sumsq) + 1e-6)); norm_out = sqrt(sumsq).
__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float* coef, float* norm_out) {
  float nrm = sqrtf(*sumsq);
  if (norm_out) *norm_out = nrm;
  float c = max_norm / (nrm + 1e-6f);
  *coef = c < 1.f ? c : 1.f;
}

}  // namespace tpb

using namespace tpb;

static AdamHyper make_hyper(float lr, float b1, float b2, float eps, float wd, int step,
                            float grad_scale, int maximize) {
  AdamHyper h;
  h.lr = lr; h.beta1 = b1; h.beta2 = b2; h.eps = eps; h.weight_decay = wd;
  h.bias_c1 = 1.f - powf(b1, (float)step);
  h.bias_c2 = 1.f - powf(b2, (float)step);
  h.grad_scale = grad_scale; h.maximize = maximize;
  return h;
}

// Overlap mode of the flat AdamW (see tpb_adamw_set_overlap).
static int g_adamw_ctas_per_sm = 0;
static bool g_adamw_max_shared = false;
static bool g_adamw_carveout_dirty = false;

// ctas_per_sm > 0 limits the grid of tpb_adamw_flat to that many CTAs per SM and max_shared != 0 lets
// them share an SM with the persistent GEMM: a memory-bound update launched on a side stream then
// trickles along under the compute-bound GEMMs of the next layer instead of holding their SMs.
// (0, 0) restores the stand-alone configuration (full grid, default carveout).
extern "C" int tpb_adamw_set_overlap(int ctas_per_sm, int max_shared) {
  g_adamw_ctas_per_sm = ctas_per_sm;
  g_adamw_max_shared = max_shared != 0;
  g_adamw_carveout_dirty = true;
  return 0;
}

extern "C" int tpb_adamw_flat(float* master, float* m, float* v, const void* grad, int grad_bf16,
                              void* model, int model_bf16, long long n, float lr, float beta1,
                              float beta2, float eps, float wd, int step, float grad_scale,
                              int maximize, const float* clip_coef, const float* found_inf,
                              void* stream) {
  TPB_NVTX("tpb_adamw_flat");
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -2;
  if ((reinterpret_cast<uintptr_t>(grad) & (grad_bf16 ? 7 : 15)) ||
      (model && (reinterpret_cast<uintptr_t>(model) & (model_bf16 ? 7 : 15))))
    return -2;
  AdamHyper h = make_hyper(lr, beta1, beta2, eps, wd, step, grad_scale, maximize);
  long long blocks = (n / 4 + 255) / 256;
  long long cap = (long long)sm_count() * (g_adamw_ctas_per_sm > 0 ? g_adamw_ctas_per_sm : 16);
  int grid = (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
  // the tail loop needs at least ceil(3/256) = 1 block; grid >= 1 always holds
  cudaStream_t s = (cudaStream_t)stream;
  if (g_adamw_carveout_dirty) {
    // In overlap mode the kernel accepts the persistent GEMM's shared-memory carveout, so that its
    // CTAs can be placed on an SM beside a GEMM CTA (an SM keeps its L1 / shared split while any CTA
    // is resident; with the default preference the next GEMM would wait for this kernel to drain).
    const int pref = g_adamw_max_shared ? (int)cudaSharedmemCarveoutMaxShared : (int)cudaSharedmemCarveoutDefault;
    cudaFuncSetAttribute(adamw_flat_kernel<__nv_bfloat16, __nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, pref);
    cudaFuncSetAttribute(adamw_flat_kernel<__nv_bfloat16, float>, cudaFuncAttributePreferredSharedMemoryCarveout, pref);
    cudaFuncSetAttribute(adamw_flat_kernel<float, __nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, pref);
    cudaFuncSetAttribute(adamw_flat_kernel<float, float>, cudaFuncAttributePreferredSharedMemoryCarveout, pref);
    g_adamw_carveout_dirty = false;
  }
#define LAUNCH(GT, MT)                                                                     \
  adamw_flat_kernel<GT, MT><<<grid, 256, 0, s>>>(master, m, v, (const GT*)grad, (MT*)model, n, h, \
                                                 clip_coef, found_inf)
  if (grad_bf16 && model_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (grad_bf16) LAUNCH(__nv_bfloat16, float);
  else if (model_bf16) LAUNCH(float, __nv_bfloat16);
  else LAUNCH(float, float);
#undef LAUNCH
  return (int)cudaGetLastError();
}

// Multi-tensor AdamW over `count` tensors given as arrays of device pointers (host arrays).
extern "C" int tpb_adamw_multi(int count, void* const* master, void* const* m, void* const* v,
                               const void* const* grad, void* const* model,
                               const long long* numel, int grad_bf16, int model_bf16, float lr,
                               float beta1, float beta2, float eps, float wd, int step,
                               float grad_scale, int maximize, const float* clip_coef,
                               const float* found_inf, void* stream) {
  TPB_NVTX("tpb_adamw_multi");
  AdamHyper h = make_hyper(lr, beta1, beta2, eps, wd, step, grad_scale, maximize);
  cudaStream_t s = (cudaStream_t)stream;
  MtaArgs a;
  int nt = 0, nb = 0;
  auto flush = [&]() -> int {
    if (nb == 0) { nt = 0; return 0; }
#define LAUNCH(GT, MT) adamw_mta_kernel<GT, MT><<<nb, 512, 0, s>>>(a, h, clip_coef, found_inf)
    if (grad_bf16 && model_bf16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (grad_bf16) LAUNCH(__nv_bfloat16, float);
    else if (model_bf16) LAUNCH(float, __nv_bfloat16);
    else LAUNCH(float, float);
#undef LAUNCH
    nt = 0; nb = 0;
    return (int)cudaGetLastError();
  };
  for (int i = 0; i < count; ++i) {
    long long n = numel[i];
    if (n <= 0) continue;
    int chunks = (int)((n + kMtaChunk - 1) / kMtaChunk);
    int c = 0;
    while (c < chunks) {
      if (nt == kMtaTensors || nb == kMtaBlocks) { int r = flush(); if (r) return r; }
      int t = nt++;
      a.master[t] = master[i]; a.m[t] = m[i]; a.v[t] = v[i]; a.grad[t] = grad[i];
      a.model[t] = model ? model[i] : nullptr; a.numel[t] = n;
      while (c < chunks && nb < kMtaBlocks) {
        a.block_tensor[nb] = (unsigned char)t;
        a.block_chunk[nb] = c++;
        ++nb;
      }
    }
  }
  return flush();
}

extern "C" int tpb_sumsq(const void* x, int is_bf16, long long n, float scale, float* out,
                         void* stream) {
  TPB_NVTX("tpb_sumsq");
  if (n <= 0) return 0;
  long long blocks = (n + 256 * 8 - 1) / (256 * 8);
  long long cap = (long long)sm_count() * 8;
  int grid = (int)(blocks < cap ? blocks : cap);
  if (is_bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, n, scale, out);
  else sumsq_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)x, n, scale, out);
  return (int)cudaGetLastError();
}

extern "C" int tpb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out,
                             void* stream) {
  TPB_NVTX("tpb_clip_coef");
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq, max_norm, coef, norm_out);
  return (int)cudaGetLastError();
}
