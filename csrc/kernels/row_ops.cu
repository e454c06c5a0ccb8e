// Memory-bound row kernels for sm_100a: RMSNorm / LayerNorm forward+backward, RoPE, SwiGLU / GELU,
// fused cross-entropy forward+backward. All use 16-byte vector accesses and fp32 math on bf16
// storage; each is sized so that one pass over HBM is the cost.
//
// Counterparts in the reference: p10/src/backend/cuda/norm/RMSNormKernels.cu:147-486,
// norm/LayerNormKernels.cu:172-1053, transformers/AttentionRopeKernels.cu:141-272,
// ActivationKernels.cu:420-520, SoftmaxKernels.cu + LossFillKernels.cu:354-470.
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int kRowThreads = 256;
constexpr int kMaxVec = 8;  // 16-byte vectors per thread kept in registers

union Vec8 {
  uint4 u;
  __nv_bfloat162 h[4];
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  Vec8 v;
  v.u = u;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(v.h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  Vec8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) v.h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v.u;
}

// Sum over the TPR threads that share a row (TPR is a power of two, 8..256).
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float* scratch /* kRowThreads/32 floats */) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o, W);
  if constexpr (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    const int wpr = TPR / 32;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[warp] = v;
    __syncthreads();
    const int first = (warp / wpr) * wpr;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < wpr; ++i) s += scratch[first + i];
    v = s;
  }
  return v;
}
template <int TPR>
__device__ __forceinline__ float row_max(float v, float* scratch) {
  constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o, W));
  if constexpr (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    const int wpr = TPR / 32;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[warp] = v;
    __syncthreads();
    const int first = (warp / wpr) * wpr;
    float s = -INFINITY;
#pragma unroll
    for (int i = 0; i < wpr; ++i) s = fmaxf(s, scratch[first + i]);
    v = s;
  }
  return v;
}

// ------------------------------------------------------------------ RMSNorm forward
// y = (x [+ res]) * rstd * w ; optionally writes the summed residual stream back (res_out).
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int rows,
                   int H, long long x_stride, long long y_stride, float eps) {
  __shared__ float scratch[kRowThreads / 32];
  constexpr int RPB = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = H / 8;
  for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += (long long)gridDim.x * RPB) {
    const long long row = row0 + threadIdx.x / TPR;
    const bool live = row < rows;
    uint4 xv[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        uint4 a = reinterpret_cast<const uint4*>(x + row * x_stride)[v];
        float f[8];
        unpack8(a, f);
        if (res) {
          float g[8];
          unpack8(reinterpret_cast<const uint4*>(res + row * (long long)H)[v], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] += g[j];
          a = pack8(f);
          unpack8(a, f);  // the normalised value is computed from the rounded stream
          if (res_out) reinterpret_cast<uint4*>(res_out + row * (long long)H)[v] = a;
        }
        xv[i] = a;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
      }
    }
    ss = row_sum<TPR>(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (live && t == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        float f[8], g[8];
        unpack8(xv[i], f);
        unpack8(reinterpret_cast<const uint4*>(w)[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = f[j] * rstd * g[j];
        reinterpret_cast<uint4*>(y + row * y_stride)[v] = pack8(f);
      }
    }
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) [+ dres]; dw partials per CTA in `dw_part`
// ([gridDim.x, H] fp32), reduced by colsum_kernel.
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_part, int rows, int H, long long x_stride,
                   long long dy_stride, long long dx_stride) {
  __shared__ float scratch[kRowThreads / 32];
  constexpr int RPB = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int sub = threadIdx.x / TPR;
  const int nvec = H / 8;
  float dwacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;

  for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += (long long)gridDim.x * RPB) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const float rstd = live ? rstd_in[row] : 0.f;
    uint4 xv[VPT], gv[VPT];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        xv[i] = reinterpret_cast<const uint4*>(x + row * x_stride)[v];
        gv[i] = reinterpret_cast<const uint4*>(dy + row * dy_stride)[v];
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf);
        unpack8(gv[i], gf);
        unpack8(reinterpret_cast<const uint4*>(w)[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float xh = xf[j] * rstd;
          dot += wf[j] * gf[j] * xh;
          dwacc[i][j] += gf[j] * xh;
        }
      }
    }
    dot = row_sum<TPR>(dot, scratch) / (float)H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[i], xf);
        unpack8(gv[i], gf);
        unpack8(reinterpret_cast<const uint4*>(w)[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (wf[j] * gf[j] - xf[j] * rstd * dot);
        if (dres) {
          float r[8];
          unpack8(reinterpret_cast<const uint4*>(dres + row * (long long)H)[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<uint4*>(dx + row * dx_stride)[v] = pack8(o);
      }
    }
  }
  // Fold the RPB sub-rows of this CTA, then write one partial row per CTA.
  float* out = dw_part + (size_t)blockIdx.x * H;
  if constexpr (RPB == 1) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) out[v * 8 + j] = dwacc[i][j];
      }
    }
  } else {
    // Several rows per CTA (small H): serialise the sub-row groups through global memory adds.
    for (int s = 0; s < RPB; ++s) {
      if (sub == s) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          int v = t + i * TPR;
          if (v < nvec) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (s == 0) out[v * 8 + j] = dwacc[i][j];
              else out[v * 8 + j] += dwacc[i][j];
            }
          }
        }
      }
      __syncthreads();
    }
  }
}

// out[c] = sum_r part[r, c]; one thread per column, coalesced across the warp.
__global__ void colsum_kernel(const float* __restrict__ part, int nrows, int H,
                              float* __restrict__ out_f32, __nv_bfloat16* __restrict__ out_bf16,
                              int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += part[(size_t)r * H + c];
  if (out_f32) out_f32[c] = accumulate ? out_f32[c] + s : s;
  if (out_bf16)
    out_bf16[c] = __float2bfloat16(accumulate ? __bfloat162float(out_bf16[c]) + s : s);
}

// ------------------------------------------------------------------ LayerNorm
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int H,
                     float eps) {
  __shared__ float scratch[kRowThreads / 32];
  constexpr int RPB = kRowThreads / TPR;
  const int t = threadIdx.x % TPR;
  const int nvec = H / 8;
  for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += (long long)gridDim.x * RPB) {
    const long long row = row0 + threadIdx.x / TPR;
    const bool live = row < rows;
    uint4 xv[VPT];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        xv[i] = reinterpret_cast<const uint4*>(x + row * (long long)H)[v];
        float f[8];
        unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += f[j];
      }
    }
    const float mean = row_sum<TPR>(s, scratch) / (float)H;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        float f[8];
        unpack8(xv[i], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += (f[j] - mean) * (f[j] - mean);
      }
    }
    const float rstd = rsqrtf(row_sum<TPR>(ss, scratch) / (float)H + eps);
    if (live && t == 0) {
      if (mean_out) mean_out[row] = mean;
      if (rstd_out) rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        float f[8], g[8], bb[8];
        unpack8(xv[i], f);
        unpack8(reinterpret_cast<const uint4*>(w)[v], g);
        if (b) unpack8(reinterpret_cast<const uint4*>(b)[v], bb);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * g[j] + (b ? bb[j] : 0.f);
        reinterpret_cast<uint4*>(y + row * (long long)H)[v] = pack8(f);
      }
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g*xhat)), g = w*dy; dw/db partial rows per CTA.
template <int TPR, int VPT>
__global__ void __launch_bounds__(kRowThreads)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                     float* __restrict__ dw_part, float* __restrict__ db_part, int rows, int H) {
  __shared__ float scratch[kRowThreads / 32];
  constexpr int RPB = kRowThreads / TPR;
  static_assert(RPB == 1 || TPR <= 128, "");
  const int t = threadIdx.x % TPR;
  const int sub = threadIdx.x / TPR;
  const int nvec = H / 8;
  float dwacc[VPT][8], dbacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = dbacc[i][j] = 0.f;
  for (long long row0 = (long long)blockIdx.x * RPB; row0 < rows; row0 += (long long)gridDim.x * RPB) {
    const long long row = row0 + sub;
    const bool live = row < rows;
    const float mean = live ? mean_in[row] : 0.f;
    const float rstd = live ? rstd_in[row] : 0.f;
    uint4 xv[VPT], gv[VPT];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        xv[i] = reinterpret_cast<const uint4*>(x + row * (long long)H)[v];
        gv[i] = reinterpret_cast<const uint4*>(dy + row * (long long)H)[v];
        float xf[8], gf[8], wf[8];
        unpack8(xv[i], xf);
        unpack8(gv[i], gf);
        unpack8(reinterpret_cast<const uint4*>(w)[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float xh = (xf[j] - mean) * rstd;
          float g = wf[j] * gf[j];
          s1 += g;
          s2 += g * xh;
          dwacc[i][j] += gf[j] * xh;
          dbacc[i][j] += gf[j];
        }
      }
    }
    s1 = row_sum<TPR>(s1, scratch) / (float)H;
    s2 = row_sum<TPR>(s2, scratch) / (float)H;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = t + i * TPR;
      if (live && v < nvec) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[i], xf);
        unpack8(gv[i], gf);
        unpack8(reinterpret_cast<const uint4*>(w)[v], wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float xh = (xf[j] - mean) * rstd;
          o[j] = rstd * (wf[j] * gf[j] - s1 - xh * s2);
        }
        reinterpret_cast<uint4*>(dx + row * (long long)H)[v] = pack8(o);
      }
    }
  }
  float* ow = dw_part + (size_t)blockIdx.x * H;
  float* ob = db_part + (size_t)blockIdx.x * H;
  for (int s = 0; s < RPB; ++s) {
    if (sub == s) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        int v = t + i * TPR;
        if (v < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (s == 0) { ow[v * 8 + j] = dwacc[i][j]; ob[v * 8 + j] = dbacc[i][j]; }
            else { ow[v * 8 + j] += dwacc[i][j]; ob[v * 8 + j] += dbacc[i][j]; }
          }
        }
      }
    }
    if (RPB > 1) __syncthreads();
  }
}

// ------------------------------------------------------------------ RoPE (in place capable)
// x viewed as [tokens, heads, D] with explicit token/head strides (elements), y likewise with its
// own strides (y == x rotates in place: each thread reads all it needs before it writes). cos/sin
// tables are fp32 [max_pos, D/2]; pos[token] optional (else token % seq_len). sign = -1 for backward.
__global__ void rope_kernel(const __nv_bfloat16* x, __nv_bfloat16* y, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const long long* __restrict__ pos,
                            long long tokens, int heads, int D, long long tok_stride,
                            long long head_stride, long long y_tok_stride, long long y_head_stride,
                            int seq_len, int interleaved, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;  // NeoX: 8 pairs per thread from both halves
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  long long total = tokens * heads * vec_per_head;
  if (idx >= total) return;
  int v = idx % vec_per_head;
  long long th = idx / vec_per_head;
  int h = th % heads;
  long long tok = th / heads;
  long long p = pos ? pos[tok] : (tok % seq_len);
  const __nv_bfloat16* base = x + tok * tok_stride + (long long)h * head_stride;
  __nv_bfloat16* obase = y + tok * y_tok_stride + (long long)h * y_head_stride;
  const float* c = cos_t + p * half;
  const float* s = sin_t + p * half;
  if (!interleaved) {
    uint4 a = reinterpret_cast<const uint4*>(base)[v];
    uint4 b = reinterpret_cast<const uint4*>(base + half)[v];
    float af[8], bf[8], oa[8], ob[8];
    unpack8(a, af);
    unpack8(b, bf);
    // cos / sin of this thread's eight pairs as four 16-byte loads (half is a multiple of 8 floats, the tables
    // are 16-byte aligned rows)
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(c + v * 8)), c1 = __ldg(reinterpret_cast<const float4*>(c + v * 8) + 1);
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(s + v * 8)), s1 = __ldg(reinterpret_cast<const float4*>(s + v * 8) + 1);
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn8[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cc = cs[j], sn = sign * sn8[j];
      oa[j] = af[j] * cc - bf[j] * sn;
      ob[j] = bf[j] * cc + af[j] * sn;
    }
    reinterpret_cast<uint4*>(obase)[v] = pack8(oa);
    reinterpret_cast<uint4*>(obase + half)[v] = pack8(ob);
  } else {
    // 16 consecutive elements = 8 (even, odd) pairs: two vectors per thread
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      uint4 a = reinterpret_cast<const uint4*>(base)[v * 2 + q];
      float f[8], o[8];
      unpack8(a, f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int pi = v * 8 + q * 4 + j;
        float cc = c[pi], sn = sign * s[pi];
        o[2 * j] = f[2 * j] * cc - f[2 * j + 1] * sn;
        o[2 * j + 1] = f[2 * j + 1] * cc + f[2 * j] * sn;
      }
      reinterpret_cast<uint4*>(obase)[v * 2 + q] = pack8(o);
    }
  }
}

// ------------------------------------------------------------------ SwiGLU / GELU
// out[r, i] = silu(gate[r, i]) * up[r, i]; gate/up given with a common row stride.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up,
                                  __nv_bfloat16* __restrict__ out, long long rows, int I,
                                  long long in_stride, const int* __restrict__ rows_dev) {
  const int nvec = I / 8;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (rows_dev) rows = min(rows, (long long)*rows_dev);  // row count known only on the device (ragged buffers)
  if (idx >= rows * nvec) return;
  long long r = idx / nvec;
  int v = idx % nvec;
  float g[8], u[8], o[8];
  unpack8(reinterpret_cast<const uint4*>(gate + r * in_stride)[v], g);
  unpack8(reinterpret_cast<const uint4*>(up + r * in_stride)[v], u);
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  reinterpret_cast<uint4*>(out + r * (long long)I)[v] = pack8(o);
}
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                  const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up,
                                  __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                                  long long rows, int I, long long in_stride,
                                  long long out_stride, const int* __restrict__ rows_dev) {
  const int nvec = I / 8;
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (rows_dev) rows = min(rows, (long long)*rows_dev);
  if (idx >= rows * nvec) return;
  long long r = idx / nvec;
  int v = idx % nvec;
  float g[8], u[8], d[8], dg[8], du[8];
  unpack8(reinterpret_cast<const uint4*>(gate + r * in_stride)[v], g);
  unpack8(reinterpret_cast<const uint4*>(up + r * in_stride)[v], u);
  unpack8(reinterpret_cast<const uint4*>(dy + r * (long long)I)[v], d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float sg = 1.f / (1.f + __expf(-g[j]));
    float silu = g[j] * sg;
    du[j] = d[j] * silu;
    dg[j] = d[j] * u[j] * (sg + silu * (1.f - sg));
  }
  reinterpret_cast<uint4*>(dgate + r * out_stride)[v] = pack8(dg);
  reinterpret_cast<uint4*>(dup + r * out_stride)[v] = pack8(du);
}

// GELU; approx = 1 selects the tanh form.
__device__ __forceinline__ float gelu_f(float x, int approx) {
  if (approx) {
    float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x));
    return 0.5f * x * (1.f + t);
  }
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}
__device__ __forceinline__ float gelu_grad_f(float x, int approx) {
  if (approx) {
    float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float t = tanhf(u);
    float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
  }
  float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
  float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  return cdf + x * pdf;
}
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                long long nvec, int approx) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nvec) return;
  float f[8];
  unpack8(reinterpret_cast<const uint4*>(x)[idx], f);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = gelu_f(f[j], approx);
  reinterpret_cast<uint4*>(y)[idx] = pack8(f);
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ dx,
                                long long nvec, int approx) {
  long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nvec) return;
  float f[8], d[8];
  unpack8(reinterpret_cast<const uint4*>(x)[idx], f);
  unpack8(reinterpret_cast<const uint4*>(dy)[idx], d);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = d[j] * gelu_grad_f(f[j], approx);
  reinterpret_cast<uint4*>(dx)[idx] = pack8(f);
}

// ------------------------------------------------------------------ cross-entropy (fwd + bwd fused)
// One CTA per row. Pass 1: online max / sum-exp over the vocabulary. Pass 2 (if dlogits):
// dlogits = (softmax - onehot) * gscale, written in place or to a separate buffer.
// loss[row] = lse - logit[target]; rows whose target == ignore_index get loss 0 / grad 0.
constexpr int kCeThreads = 1024;
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                     float* __restrict__ loss, float* __restrict__ lse_out,
                     __nv_bfloat16* __restrict__ dlogits, int V, long long stride,
                     long long ignore_index, float gscale) {
  __shared__ float sm[kCeThreads / 32];
  __shared__ float ss[kCeThreads / 32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* lr = logits + row * stride;
  const long long tgt = target[row];
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    float f = __bfloat162float(lr[i]);
    float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  // block combine of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, m, o);
    float os = __shfl_xor_sync(0xffffffffu, s, o);
    float nm = fmaxf(m, om);
    s = (nm == -INFINITY) ? 0.f : s * __expf(m - nm) + os * __expf(om - nm);
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = s; }
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int i = 0; i < kCeThreads / 32; ++i) gm = fmaxf(gm, sm[i]);
  float gs = 0.f;
#pragma unroll
  for (int i = 0; i < kCeThreads / 32; ++i)
    gs += (sm[i] == -INFINITY) ? 0.f : ss[i] * __expf(sm[i] - gm);
  const float lse = gm + __logf(gs);
  const bool ignored = (tgt == ignore_index) || !TPB_DBG_CHECK(tgt >= 0 && tgt < V, 43);
  if (threadIdx.x == 0) {
    if (lse_out) lse_out[row] = lse;
    if (loss) loss[row] = ignored ? 0.f : lse - __bfloat162float(lr[tgt]);
  }
  if (!dlogits) return;
  __nv_bfloat16* dr = dlogits + row * stride;
  const float gsc = ignored ? 0.f : gscale;
  for (int v = threadIdx.x; v < nvec; v += kCeThreads) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pr = __expf(f[j] - lse);
      if ((long long)(v * 8 + j) == tgt) pr -= 1.f;
      f[j] = pr * gsc;
    }
    reinterpret_cast<uint4*>(dr)[v] = pack8(f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    float pr = __expf(__bfloat162float(lr[i]) - lse);
    if (i == tgt) pr -= 1.f;
    dr[i] = __float2bfloat16(pr * gsc);
  }
}

// Backward from a saved log-sum-exp: dlogits = (exp(l - lse) - onehot) * g, where
// g = g_scalar[0] * scale[0] (either may be null) or g_rows[row]. Grid (chunks, rows).
__global__ void __launch_bounds__(256)
cross_entropy_bwd_kernel(const __nv_bfloat16* __restrict__ logits,
                         const long long* __restrict__ target, const float* __restrict__ lse_in,
                         __nv_bfloat16* __restrict__ dlogits, const float* __restrict__ g_scalar,
                         const float* __restrict__ scale, const float* __restrict__ g_rows, int V,
                         long long stride, long long ignore_index) {
  const long long row = blockIdx.y;
  const long long tgt = target[row];
  const bool ignored = (tgt == ignore_index) || !TPB_DBG_CHECK(tgt >= 0 && tgt < V, 43);
  float g = g_rows ? g_rows[row] : 1.f;
  if (g_scalar) g *= *g_scalar;
  if (scale) g *= *scale;
  if (ignored) g = 0.f;
  const float lse = lse_in[row];
  const __nv_bfloat16* lr = logits + row * stride;
  __nv_bfloat16* dr = dlogits + row * stride;
  const int nvec = V / 8;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += gridDim.x * blockDim.x) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(lr)[v], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float pr = __expf(f[j] - lse);
      if ((long long)(v * 8 + j) == tgt) pr -= 1.f;
      f[j] = pr * g;
    }
    reinterpret_cast<uint4*>(dr)[v] = pack8(f);
  }
  if (blockIdx.x == 0) {
    for (int i = nvec * 8 + threadIdx.x; i < V; i += blockDim.x) {
      float pr = __expf(__bfloat162float(lr[i]) - lse);
      if (i == tgt) pr -= 1.f;
      dr[i] = __float2bfloat16(pr * g);
    }
  }
}

// ------------------------------------------------------------------ launch helpers
static int pick_tpr(int H) {
  int nvec = H / 8;
  return nvec <= 16 ? 16 : (nvec <= 256 ? 128 : 256);
}
static int pick_vpt(int H, int tpr) {
  int need = (H / 8 + tpr - 1) / tpr;
  int v = 1;
  while (v < need) v <<= 1;
  return v;
}
int row_grid(int rows, int tpr) {
  int rpb = kRowThreads / tpr;
  long long blocks = ((long long)rows + rpb - 1) / rpb;
  long long cap = (long long)sm_count() * 8;
  return (int)(blocks < cap ? blocks : cap);
}

#define TPB_VPT_SWITCH(vpt, ...)                          \
  switch (vpt) {                                          \
    case 1: { constexpr int VPT = 1; __VA_ARGS__; } break; \
    case 2: { constexpr int VPT = 2; __VA_ARGS__; } break; \
    case 4: { constexpr int VPT = 4; __VA_ARGS__; } break; \
    case 8: { constexpr int VPT = 8; __VA_ARGS__; } break; \
    default: return -2;                                   \
  }
#define TPB_ROW_SWITCH(tpr, vpt, ...)                                          \
  switch (tpr) {                                                               \
    case 16: { constexpr int TPR = 16; TPB_VPT_SWITCH(vpt, __VA_ARGS__) } break;   \
    case 128: { constexpr int TPR = 128; TPB_VPT_SWITCH(vpt, __VA_ARGS__) } break; \
    case 256: { constexpr int TPR = 256; TPB_VPT_SWITCH(vpt, __VA_ARGS__) } break; \
    default: return -2;                                                        \
  }

}  // namespace tpb

using namespace tpb;

extern "C" int tpb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out,
                               float* rstd, int rows, int H, long long x_stride,
                               long long y_stride, float eps, void* stream) {
  TPB_NVTX("tpb_rmsnorm_fwd");
  if (H % 8 || H > 256 * kMaxVec * 8) return -2;
  if (rows <= 0) return 0;
  int tpr = pick_tpr(H);
  int grid = ((long long)rows + kRowThreads / tpr - 1) / (kRowThreads / tpr);
  TPB_ROW_SWITCH(tpr, pick_vpt(H, tpr), (rmsnorm_fwd_kernel<TPR, VPT><<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)res,
                          (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (__nv_bfloat16*)res_out, rstd,
                          rows, H, x_stride, y_stride, eps)));
  return (int)cudaGetLastError();
}

extern "C" int tpb_rmsnorm_bwd_grid(int rows, int H) {
  if (H % 8 || H > 256 * kMaxVec * 8) return -2;
  int tpr = pick_tpr(H);
  int g = row_grid(rows, tpr);
  // 4 CTAs of 62-64 registers x 256 threads fit an SM; each CTA works through its rows one after the
  // other (load, row reduction, store), so resident CTAs are what hides the memory latency
  int cap = sm_count() * 4;
  return g < cap ? g : cap;
}

// dw_part must hold tpb_rmsnorm_bwd_grid(rows, H) * H floats.
extern "C" int tpb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                               const void* dres, void* dx, float* dw_part, float* dw_f32,
                               void* dw_bf16, int dw_accumulate, int rows, int H,
                               long long x_stride, long long dy_stride, long long dx_stride,
                               void* stream) {
  TPB_NVTX("tpb_rmsnorm_bwd");
  if (H % 8 || H > 256 * kMaxVec * 8) return -2;
  if (rows <= 0) return 0;
  int tpr = pick_tpr(H);
  int grid = tpb_rmsnorm_bwd_grid(rows, H);
  TPB_ROW_SWITCH(tpr, pick_vpt(H, tpr), (rmsnorm_bwd_kernel<TPR, VPT><<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
                          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                          (__nv_bfloat16*)dx, dw_part, rows, H, x_stride, dy_stride, dx_stride)));
  colsum_kernel<<<(H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      dw_part, grid, H, dw_f32, (__nv_bfloat16*)dw_bf16, dw_accumulate);
  return (int)cudaGetLastError();
}

extern "C" int tpb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                                 float* rstd, int rows, int H, float eps, void* stream) {
  TPB_NVTX("tpb_layernorm_fwd");
  if (H % 8 || H > 256 * kMaxVec * 8) return -2;
  if (rows <= 0) return 0;
  int tpr = pick_tpr(H);
  int grid = ((long long)rows + kRowThreads / tpr - 1) / (kRowThreads / tpr);
  TPB_ROW_SWITCH(tpr, pick_vpt(H, tpr), (layernorm_fwd_kernel<TPR, VPT><<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                          (const __nv_bfloat16*)b, (__nv_bfloat16*)y, mean, rstd, rows, H, eps)));
  return (int)cudaGetLastError();
}

// dw_part / db_part: tpb_rmsnorm_bwd_grid(rows, H) * H floats each.
extern "C" int tpb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                                 const float* rstd, void* dx, float* dw_part, float* db_part,
                                 float* dw_f32, void* dw_bf16, float* db_f32, void* db_bf16,
                                 int accumulate, int rows, int H, void* stream) {
  TPB_NVTX("tpb_layernorm_bwd");
  if (H % 8 || H > 256 * kMaxVec * 8) return -2;
  if (rows <= 0) return 0;
  int tpr = pick_tpr(H);
  int grid = tpb_rmsnorm_bwd_grid(rows, H);
  TPB_ROW_SWITCH(tpr, pick_vpt(H, tpr), (layernorm_bwd_kernel<TPR, VPT><<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
                          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)w, mean, rstd, (__nv_bfloat16*)dx, dw_part, db_part,
                          rows, H)));
  colsum_kernel<<<(H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      dw_part, grid, H, dw_f32, (__nv_bfloat16*)dw_bf16, accumulate);
  colsum_kernel<<<(H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      db_part, grid, H, db_f32, (__nv_bfloat16*)db_bf16, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int tpb_rope_out(const void* x, void* y, const float* cos_t, const float* sin_t,
                            const long long* pos, long long tokens, int heads, int D,
                            long long tok_stride, long long head_stride, long long y_tok_stride,
                            long long y_head_stride, int seq_len, int interleaved, int backward,
                            void* stream) {
  TPB_NVTX("tpb_rope_out");
  if (D % 16 || tok_stride % 8 || head_stride % 8 || y_tok_stride % 8 || y_head_stride % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(cos_t) |
       reinterpret_cast<uintptr_t>(sin_t)) & 15)
    return -2;
  long long total = tokens * heads * (D / 16);
  if (total <= 0) return 0;
  int grid = (int)((total + 255) / 256);
  rope_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, cos_t, sin_t, pos, tokens, heads, D, tok_stride,
      head_stride, y_tok_stride, y_head_stride, seq_len, interleaved, backward ? -1.f : 1.f);
  return (int)cudaGetLastError();
}
extern "C" int tpb_rope(void* x, const float* cos_t, const float* sin_t, const long long* pos,
                        long long tokens, int heads, int D, long long tok_stride,
                        long long head_stride, int seq_len, int interleaved, int backward,
                        void* stream) {
  TPB_NVTX("tpb_rope");
  return tpb_rope_out(x, x, cos_t, sin_t, pos, tokens, heads, D, tok_stride, head_stride, tok_stride,
                      head_stride, seq_len, interleaved, backward, stream);
}

// rows_dev (optional): device word with the number of rows actually in use (<= rows); rows beyond it
// are neither read nor written (expert buffers are sized for the worst case, filled to a
// data-dependent row).
extern "C" int tpb_swiglu_fwd_n(const void* gate, const void* up, void* out, long long rows, int I,
                                long long in_stride, const int* rows_dev, void* stream) {
  TPB_NVTX("tpb_swiglu_fwd_n");
  if (I % 8 || in_stride % 8) return -2;
  long long total = rows * (I / 8);
  if (total <= 0) return 0;
  swiglu_fwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, (__nv_bfloat16*)out, rows, I,
      in_stride, rows_dev);
  return (int)cudaGetLastError();
}
extern "C" int tpb_swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int I,
                              long long in_stride, void* stream) {
  TPB_NVTX("tpb_swiglu_fwd");
  return tpb_swiglu_fwd_n(gate, up, out, rows, I, in_stride, nullptr, stream);
}
extern "C" int tpb_swiglu_bwd_n(const void* dy, const void* gate, const void* up, void* dgate,
                                void* dup, long long rows, int I, long long in_stride,
                                long long out_stride, const int* rows_dev, void* stream) {
  TPB_NVTX("tpb_swiglu_bwd_n");
  if (I % 8 || in_stride % 8 || out_stride % 8) return -2;
  long long total = rows * (I / 8);
  if (total <= 0) return 0;
  swiglu_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
      (__nv_bfloat16*)dgate, (__nv_bfloat16*)dup, rows, I, in_stride, out_stride, rows_dev);
  return (int)cudaGetLastError();
}
extern "C" int tpb_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate,
                              void* dup, long long rows, int I, long long in_stride,
                              long long out_stride, void* stream) {
  TPB_NVTX("tpb_swiglu_bwd");
  return tpb_swiglu_bwd_n(dy, gate, up, dgate, dup, rows, I, in_stride, out_stride, nullptr, stream);
}
extern "C" int tpb_gelu_fwd(const void* x, void* y, long long n, int approx, void* stream) {
  TPB_NVTX("tpb_gelu_fwd");
  if (n % 8) return -2;
  if (n <= 0) return 0;
  gelu_fwd_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / 8, approx);
  return (int)cudaGetLastError();
}
extern "C" int tpb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int approx,
                            void* stream) {
  TPB_NVTX("tpb_gelu_bwd");
  if (n % 8) return -2;
  if (n <= 0) return 0;
  gelu_bwd_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (__nv_bfloat16*)dx, n / 8, approx);
  return (int)cudaGetLastError();
}

extern "C" int tpb_cross_entropy(const void* logits, const long long* target, float* loss,
                                 float* lse, void* dlogits, long long rows, int V, long long stride,
                                 long long ignore_index, float gscale, void* stream) {
  TPB_NVTX("tpb_cross_entropy");
  if (stride % 8) return -2;
  if (rows <= 0) return 0;
  cross_entropy_kernel<<<(unsigned)rows, kCeThreads, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, target, loss, lse, (__nv_bfloat16*)dlogits, V, stride,
      ignore_index, gscale);
  return (int)cudaGetLastError();
}

extern "C" int tpb_cross_entropy_bwd(const void* logits, const long long* target, const float* lse,
                                     void* dlogits, const float* g_scalar, const float* scale,
                                     const float* g_rows, long long rows, int V, long long stride,
                                     long long ignore_index, void* stream) {
  TPB_NVTX("tpb_cross_entropy_bwd");
  if (stride % 8) return -2;
  if (rows <= 0) return 0;
  int chunks = (V / 8 + 256 * 4 - 1) / (256 * 4);
  if (chunks < 1) chunks = 1;
  dim3 grid(chunks, (unsigned)rows);
  cross_entropy_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)logits, target, lse, (__nv_bfloat16*)dlogits, g_scalar, scale, g_rows,
      V, stride, ignore_index);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ allocation-free variant
#include "tpb_noalloc.h"

// Scratch for tpb_rmsnorm_bwd_noalloc: per-block partial sums of dw. Lives in every device
// that loads this library for the life of the process.
static __device__ __align__(256) float g_noalloc_rms_scratch[TPB_NOALLOC_RMSNORM_MAX_FLOATS];

namespace {
constexpr int kNoAllocMaxDevices = 64;
float* g_noalloc_scratch_ptr[kNoAllocMaxDevices] = {};
}  // namespace

extern "C" const char* tpb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case TPB_NOALLOC_TOO_LARGE:
      return "problem exceeds the built-in scratch (H <= 8192 and at most 296 blocks are supported)";
    case TPB_NOALLOC_BAD_ARGS: return "H must be a positive multiple of 8 and strides multiples of 8";
    case TPB_NOALLOC_NO_SYMBOL: return "could not obtain the device address of the built-in scratch";
    default: return code > 0 ? "CUDA error (see cudaGetErrorString)" : "unknown error";
  }
}

extern "C" int tpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w,
                                       const float* rstd, const void* dres, void* dx, float* dw_f32,
                                       void* dw_bf16, int dw_accumulate, int rows, int H,
                                       long long x_stride, long long dy_stride, long long dx_stride,
                                       void* stream) {
  TPB_NVTX("tpb_rmsnorm_bwd_noalloc");
  if (H <= 0 || H % 8 || x_stride % 8 || dy_stride % 8 || dx_stride % 8) return TPB_NOALLOC_BAD_ARGS;
  if (H > TPB_NOALLOC_RMSNORM_MAX_H) return TPB_NOALLOC_TOO_LARGE;
  if (rows <= 0) return 0;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoAllocMaxDevices) return TPB_NOALLOC_NO_SYMBOL;
  // First call on this device: the array's name is only a host-side handle, the kernel needs
  // the address the symbol has on the current device.
  float* scratch = g_noalloc_scratch_ptr[dev];
  if (!scratch) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_rms_scratch);
    if (e != cudaSuccess || !p) return TPB_NOALLOC_NO_SYMBOL;
    scratch = static_cast<float*>(p);
    g_noalloc_scratch_ptr[dev] = scratch;
  }
  const int tpr = pick_tpr(H);
  int grid = tpb_rmsnorm_bwd_grid(rows, H);
  if (grid > TPB_NOALLOC_RMSNORM_MAX_BLOCKS) grid = TPB_NOALLOC_RMSNORM_MAX_BLOCKS;
  if ((long long)grid * H > (long long)TPB_NOALLOC_RMSNORM_MAX_FLOATS) return TPB_NOALLOC_TOO_LARGE;
  TPB_ROW_SWITCH(tpr, pick_vpt(H, tpr), (rmsnorm_bwd_kernel<TPR, VPT><<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
                          (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,
                          (__nv_bfloat16*)dx, scratch, rows, H, x_stride, dy_stride, dx_stride)));
  colsum_kernel<<<(H + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      scratch, grid, H, dw_f32, (__nv_bfloat16*)dw_bf16, dw_accumulate);
  return (int)cudaGetLastError();
}
