// Multi-tensor SGD / Adagrad / RMSprop steps and the AMP kernels (unscale with non-finite check,
// loss-scale update) for sm_100a: one launch covers up to 48 tensors, fp32 state and fp32 (master)
// weights, optional bf16 parameter emit in the same pass, gradients in bf16 or fp32.
//
// Counterparts in the reference: p10/include/OptimizerMTA.cuh:438 (SGD), :847 (Adagrad), :988
// (RMSprop); p10/src/backend/cuda/AmpKernels.cu:63 (unscale + non-finite check), :95 (scale update).
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

enum : int { kOptSGD = 0, kOptAdagrad = 1, kOptRMSprop = 2 };
enum : int { kFlagNesterov = 1, kFlagMaximize = 2, kFlagCentered = 4, kFlagFirstStep = 8, kFlagMomentum = 16 };

struct OptHyper {
  int algo, flags;
  float lr, weight_decay, a, b, eps, grad_scale;
};

constexpr int kOptTensors = 48;
constexpr int kOptBlocks = 640;
constexpr int kOptChunk = 65536;
struct OptArgs {
  void* param[kOptTensors];
  void* s1[kOptTensors];
  void* s2[kOptTensors];
  void* s3[kOptTensors];
  const void* grad[kOptTensors];
  void* model[kOptTensors];
  long long numel[kOptTensors];
  unsigned char block_tensor[kOptBlocks];
  int block_chunk[kOptBlocks];
};

template <typename GradT>
__global__ void __launch_bounds__(512)
optim_mta_kernel(const __grid_constant__ OptArgs a, OptHyper h, const float* __restrict__ found_inf) {
  if (found_inf && *found_inf != 0.f) return;
  const int t = a.block_tensor[blockIdx.x];
  const long long start = (long long)a.block_chunk[blockIdx.x] * kOptChunk;
  const long long n = a.numel[t];
  const long long end = start + kOptChunk < n ? start + kOptChunk : n;
  float* p = reinterpret_cast<float*>(a.param[t]);
  float* s1 = reinterpret_cast<float*>(a.s1[t]);
  float* s2 = reinterpret_cast<float*>(a.s2[t]);
  float* s3 = reinterpret_cast<float*>(a.s3[t]);
  const GradT* grad = reinterpret_cast<const GradT*>(a.grad[t]);
  __nv_bfloat16* model = reinterpret_cast<__nv_bfloat16*>(a.model[t]);
  for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
    float g;
    if constexpr (sizeof(GradT) == 2) g = __bfloat162float(grad[i]);
    else g = grad[i];
    g *= h.grad_scale;
    if (h.flags & kFlagMaximize) g = -g;
    float w = p[i];
    g += h.weight_decay * w;
    if (h.algo == kOptSGD) {
      if (h.flags & kFlagMomentum) {
        float buf = (h.flags & kFlagFirstStep) ? g : h.a * s1[i] + (1.f - h.b) * g;
        s1[i] = buf;
        g = (h.flags & kFlagNesterov) ? g + h.a * buf : buf;
      }
      w -= h.lr * g;
    } else if (h.algo == kOptAdagrad) {
      const float sum = s1[i] + g * g;
      s1[i] = sum;
      w -= h.lr * g / (sqrtf(sum) + h.eps);
    } else {
      const float sq = h.a * s1[i] + (1.f - h.a) * g * g;
      s1[i] = sq;
      float avg;
      if (h.flags & kFlagCentered) {
        const float ga = h.a * s3[i] + (1.f - h.a) * g;
        s3[i] = ga;
        avg = sqrtf(fmaxf(sq - ga * ga, 0.f)) + h.eps;
      } else {
        avg = sqrtf(sq) + h.eps;
      }
      if (h.flags & kFlagMomentum) {
        const float buf = h.b * s2[i] + g / avg;
        s2[i] = buf;
        w -= h.lr * buf;
      } else {
        w -= h.lr * g / avg;
      }
    }
    p[i] = w;
    if (model) model[i] = __float2bfloat16(w);
  }
}

// grads *= *inv_scale (in place); *found_inf = 1 if any value is inf or nan.
template <typename T>
__global__ void __launch_bounds__(512)
amp_unscale_kernel(const __grid_constant__ OptArgs a, const float* __restrict__ inv_scale, float* __restrict__ found_inf) {
  const int t = a.block_tensor[blockIdx.x];
  const long long start = (long long)a.block_chunk[blockIdx.x] * kOptChunk;
  const long long n = a.numel[t];
  const long long end = start + kOptChunk < n ? start + kOptChunk : n;
  T* g = reinterpret_cast<T*>(a.param[t]);
  const float s = *inv_scale;
  bool bad = false;
  for (long long i = start + threadIdx.x; i < end; i += blockDim.x) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(g[i]);
    else v = g[i];
    bad |= !isfinite(v);
    v *= s;
    if constexpr (sizeof(T) == 2) g[i] = __float2bfloat16(v);
    else g[i] = v;
  }
  if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *found_inf = 1.f;
}

// One thread: the dynamic loss scale after a step. found_inf != 0: scale *= backoff, tracker = 0;
// otherwise tracker += 1 and, when it reaches the interval, scale *= growth (if still finite).
__global__ void amp_update_scale_kernel(float* scale, int* growth_tracker, const float* found_inf, float growth,
                                        float backoff, int interval) {
  if (*found_inf != 0.f) {
    *scale *= backoff;
    *growth_tracker = 0;
  } else {
    const int k = *growth_tracker + 1;
    if (k == interval) {
      const float ns = *scale * growth;
      if (isfinite(ns)) *scale = ns;
      *growth_tracker = 0;
    } else {
      *growth_tracker = k;
    }
  }
}

template <typename Launch>
static int for_each_batch(int count, void* const* p, void* const* s1, void* const* s2, void* const* s3,
                          const void* const* grad, void* const* model, const long long* numel, Launch launch) {
  OptArgs a;
  int nt = 0, nb = 0;
  auto flush = [&]() -> int {
    if (nb == 0) { nt = 0; return 0; }
    int r = launch(a, nb);
    nt = nb = 0;
    return r;
  };
  for (int i = 0; i < count; ++i) {
    const long long n = numel[i];
    if (n <= 0) continue;
    const int chunks = (int)((n + kOptChunk - 1) / kOptChunk);
    int c = 0;
    while (c < chunks) {
      if (nt == kOptTensors || nb == kOptBlocks) { int r = flush(); if (r) return r; }
      const int t = nt++;
      a.param[t] = p[i];
      a.s1[t] = s1 ? s1[i] : nullptr; a.s2[t] = s2 ? s2[i] : nullptr; a.s3[t] = s3 ? s3[i] : nullptr;
      a.grad[t] = grad ? grad[i] : nullptr; a.model[t] = model ? model[i] : nullptr; a.numel[t] = n;
      while (c < chunks && nb < kOptBlocks) {
        a.block_tensor[nb] = (unsigned char)t;
        a.block_chunk[nb] = c++;
        ++nb;
      }
    }
  }
  return flush();
}

}  // namespace tpb

using namespace tpb;

// One step of SGD (algo 0: a = momentum, b = dampening, flags nesterov / maximize / first step /
// momentum), Adagrad (1: lr already decayed by the caller) or RMSprop (2: a = alpha, b = momentum,
// flags centered / momentum; s1 = square average, s2 = momentum buffer, s3 = gradient average) over
// `count` tensors given as host arrays of device pointers. param: fp32 weights (the master copy of
// bf16 parameters, whose bf16 values are written to `model` when it is given); state: fp32.
extern "C" int tpb_optim_multi(int algo, int flags, int count, void* const* param, void* const* s1,
                               void* const* s2, void* const* s3, const void* const* grad, void* const* model,
                               const long long* numel, int grad_bf16, float lr, float weight_decay, float a,
                               float b, float eps, float grad_scale, const float* found_inf, void* stream) {
  TPB_NVTX("tpb_optim_multi");
  if (algo < 0 || algo > 2) return -2;
  OptHyper h;
  h.algo = algo; h.flags = flags; h.lr = lr; h.weight_decay = weight_decay; h.a = a; h.b = b; h.eps = eps;
  h.grad_scale = grad_scale;
  cudaStream_t s = (cudaStream_t)stream;
  return for_each_batch(count, param, s1, s2, s3, grad, model, numel, [&](const OptArgs& args, int nb) {
    if (grad_bf16) optim_mta_kernel<__nv_bfloat16><<<nb, 512, 0, s>>>(args, h, found_inf);
    else optim_mta_kernel<float><<<nb, 512, 0, s>>>(args, h, found_inf);
    return (int)cudaGetLastError();
  });
}

// grads[i] *= *inv_scale for every tensor; *found_inf is set to 1 when a gradient holds inf or nan
// (the caller zeroes it before the first call of a step).
extern "C" int tpb_amp_unscale_multi(int count, void* const* grads, const long long* numel, int is_bf16,
                                     const float* inv_scale, float* found_inf, void* stream) {
  TPB_NVTX("tpb_amp_unscale_multi");
  cudaStream_t s = (cudaStream_t)stream;
  return for_each_batch(count, grads, nullptr, nullptr, nullptr, nullptr, nullptr, numel,
                        [&](const OptArgs& args, int nb) {
    if (is_bf16) amp_unscale_kernel<__nv_bfloat16><<<nb, 512, 0, s>>>(args, inv_scale, found_inf);
    else amp_unscale_kernel<float><<<nb, 512, 0, s>>>(args, inv_scale, found_inf);
    return (int)cudaGetLastError();
  });
}

extern "C" int tpb_amp_update_scale(float* scale, int* growth_tracker, const float* found_inf, float growth_factor,
                                    float backoff_factor, int growth_interval, void* stream) {
  TPB_NVTX("tpb_amp_update_scale");
  amp_update_scale_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(scale, growth_tracker, found_inf, growth_factor,
                                                              backoff_factor, growth_interval);
  return (int)cudaGetLastError();
}
