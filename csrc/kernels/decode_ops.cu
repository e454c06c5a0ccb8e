// Token-level kernels around the transformer body: embedding gather / scatter-add, KV-cache
// append (contiguous and paged) and top-k / top-p sampling.
//
// Capability reference: p10/src/backend/cuda/EmbeddingKernels.cu (gather + dense backward),
// SamplingKernels.cu:350 (top-k / top-p sampling), tensorplay/nn/cache.py:51-457 (cache layouts).
#include <float.h>

#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {
namespace {

// ------------------------------------------------------------------ embedding
// out[i, :] = table[ids[i], :]; one warp per 512-byte slice of a row, 16-byte accesses.
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* __restrict__ out, long long n, int H, long long V) {
  const int vec_per_row = H / 8;
  const long long total = n * vec_per_row;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vec_per_row;
    const int c = (int)(i - r * vec_per_row);
    long long id = ids[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (TPB_DBG_CHECK(id >= 0 && id < V, 40)) v = __ldg(reinterpret_cast<const uint4*>(table + id * H) + c);
    reinterpret_cast<uint4*>(out + r * H)[c] = v;
  }
}

// dW[ids[i], :] += dy[i, :]: packed bf16x2 (or fp32) reductions performed by the L2.
template <bool F32>
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                     void* __restrict__ dw, long long n, int H, long long V) {
  const int pairs = H / 2;
  const long long total = n * pairs;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / pairs;
    const int c = (int)(i - r * pairs);
    const long long id = ids[r];
    if (!TPB_DBG_CHECK(id >= 0 && id < V, 41)) continue;
    const __nv_bfloat162 g = reinterpret_cast<const __nv_bfloat162*>(dy + r * H)[c];
    if (F32) {
      float* d = static_cast<float*>(dw) + id * H + 2 * c;
      const float2 f = __bfloat1622float2(g);
      atomicAdd(d, f.x);
      atomicAdd(d + 1, f.y);
    } else {
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(dw) + id * H) + c, g);
    }
  }
}

// ------------------------------------------------------------------ KV-cache append
// src [B, T, H, D] (strided) -> cache rows. Contiguous cache: row (b, pos[b] + t); paged cache:
// physical block = table[b, (pos + t) / block], row inside the block = (pos + t) % block.
struct KvAppendParams {
  const __nv_bfloat16* src;
  __nv_bfloat16* dst;
  const int* pos;          // [B] first position to write, or null (pos0 for all)
  const int* block_table;  // [B, max_blocks] or null
  int pos0, B, T, H, D, block, max_blocks;
  long long s_b, s_t, s_h;        // source strides (elements)
  long long d_b, d_t, d_h;        // destination strides: batch (or block), token, head
};

__global__ void __launch_bounds__(256) kv_append_kernel(const KvAppendParams p) {
  const int vec = p.D / 8;
  const long long total = (long long)p.B * p.T * p.H * vec;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int c = (int)(i % vec);
    long long r = i / vec;
    const int h = (int)(r % p.H); r /= p.H;
    const int t = (int)(r % p.T);
    const int b = (int)(r / p.T);
    const int at = (p.pos ? p.pos[b] : p.pos0) + t;
    long long off;
    if (p.block_table) {
      const int blk = at / p.block;
      if (!TPB_DBG_CHECK(blk < p.max_blocks, 42)) continue;
      const int phys = p.block_table[(long long)b * p.max_blocks + blk];
      if (phys < 0) continue;
      off = (long long)phys * p.d_b + (long long)(at % p.block) * p.d_t;
    } else {
      off = (long long)b * p.d_b + (long long)at * p.d_t;
    }
    const uint4 v = *(reinterpret_cast<const uint4*>(p.src + b * p.s_b + t * p.s_t + h * p.s_h) + c);
    *(reinterpret_cast<uint4*>(p.dst + off + h * p.d_h) + c) = v;
  }
}

// ------------------------------------------------------------------ decode-step QKV preparation
// One token per sequence: qkv [B, Hq + 2 Hkv, D] packed. Rotates the Hq query heads into q_out
// [B, Hq, D], rotates the Hkv key heads straight into the key cache at row pos[b], and copies the
// value heads into the value cache at the same row: rotation and both cache appends in one launch.
// NeoX (half-split) rotation; cos/sin are fp32 [max_pos, D / 2]. A position outside the cache or the
// tables is skipped (and reported by the debug build).
struct DecodeQkvParams {
  const __nv_bfloat16* qkv;
  __nv_bfloat16* q_out;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  const float* cos_t;
  const float* sin_t;
  const int* pos;
  int B, Hq, Hkv, D, cap, max_pos;
  long long qkv_b;             // batch stride of qkv (elements)
  long long c_b, c_t, c_h;     // cache strides: batch, token, head
};

__device__ __forceinline__ void unpack8_bf16(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8_bf16(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

__global__ void __launch_bounds__(256) decode_qkv_prep_kernel(const DecodeQkvParams p) {
  const int half = p.D / 2, vec = half / 8;          // a thread: 8 elements of each half of one head
  const int heads = p.Hq + 2 * p.Hkv;
  const long long total = (long long)p.B * heads * vec;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int c = (int)(i % vec);
    long long r = i / vec;
    const int h = (int)(r % heads);
    const int b = (int)(r / heads);
    const int at = p.pos[b];
    if (!TPB_DBG_CHECK(at >= 0 && at < p.cap && at < p.max_pos, 44)) continue;
    const __nv_bfloat16* src = p.qkv + b * p.qkv_b + (long long)h * p.D;
    uint4 lo = reinterpret_cast<const uint4*>(src)[c];
    uint4 hi = reinterpret_cast<const uint4*>(src + half)[c];
    __nv_bfloat16* dst;
    if (h < p.Hq) dst = p.q_out + ((long long)b * p.Hq + h) * p.D;
    else if (h < p.Hq + p.Hkv) dst = p.k_cache + b * p.c_b + (long long)at * p.c_t + (long long)(h - p.Hq) * p.c_h;
    else dst = p.v_cache + b * p.c_b + (long long)at * p.c_t + (long long)(h - p.Hq - p.Hkv) * p.c_h;
    if (h < p.Hq + p.Hkv) {
      float a[8], bb[8], oa[8], ob[8];
      unpack8_bf16(lo, a);
      unpack8_bf16(hi, bb);
      const float* cs = p.cos_t + (long long)at * half + c * 8;
      const float* sn = p.sin_t + (long long)at * half + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        oa[j] = a[j] * cs[j] - bb[j] * sn[j];
        ob[j] = bb[j] * cs[j] + a[j] * sn[j];
      }
      lo = pack8_bf16(oa);
      hi = pack8_bf16(ob);
    }
    reinterpret_cast<uint4*>(dst)[c] = lo;
    reinterpret_cast<uint4*>(dst + half)[c] = hi;
  }
}

// ------------------------------------------------------------------ sampling
// One CTA per row. The support is found without sorting: a 32-step radix descent over the
// order-preserving integer image of the logits gives the exact k-th largest value (top-k) and
// the smallest value whose strictly-larger mass is <= top_p (nucleus); the token is then drawn
// by inverse CDF in index order from the caller's uniform number.
constexpr int kSampleThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__device__ __forceinline__ T block_sum(T v, T* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  T t = red[threadIdx.x & 31];
  if ((threadIdx.x & 31) >= (blockDim.x >> 5)) t = T(0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -FLT_MAX;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

template <typename TL>
__device__ __forceinline__ float load_logit(const TL* row, int i, float inv_temp);
template <>
__device__ __forceinline__ float load_logit<float>(const float* row, int i, float inv_temp) {
  return row[i] * inv_temp;
}
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* row, int i, float inv_temp) {
  return __bfloat162float(row[i]) * inv_temp;
}

template <typename TL>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const TL* __restrict__ logits, const float* __restrict__ uniform,
              long long* __restrict__ out, float* __restrict__ out_logit_thresh, int V,
              long long row_stride, float inv_temp, int top_k, float top_p) {
  __shared__ float redf[32];
  __shared__ int redi[32];
  __shared__ float scan[kSampleThreads / 32];
  __shared__ int s_pick;
  const TL* row = logits + (long long)blockIdx.x * row_stride;
  const int tid = threadIdx.x;

  float mx = -FLT_MAX;
  for (int i = tid; i < V; i += kSampleThreads) mx = fmaxf(mx, load_logit(row, i, inv_temp));
  mx = block_max(mx, redf);

  // top-k: largest key t with count(key >= t) >= k
  uint32_t kth = 0;
  if (top_k > 0 && top_k < V) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = kth | (1u << bit);
      int cnt = 0;
      for (int i = tid; i < V; i += kSampleThreads) cnt += order_key(load_logit(row, i, inv_temp)) >= cand;
      cnt = block_sum<int>(cnt, redi);
      if (cnt >= top_k) kth = cand;
    }
  }
  // softmax mass of the top-k support
  float z = 0.f;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float x = load_logit(row, i, inv_temp);
    if (order_key(x) >= kth) z += __expf(x - mx);
  }
  z = block_sum<float>(z, redf);

  // nucleus: smallest key t with mass(key > t) <= top_p * z; the support becomes key >= t
  uint32_t thr = kth;
  if (top_p < 1.f) {
    const float budget = top_p * z;
    uint32_t t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = t | ((1u << bit) - 1u);  // largest value of the lower half
      float above = 0.f;
      for (int i = tid; i < V; i += kSampleThreads) {
        const float x = load_logit(row, i, inv_temp);
        const uint32_t key = order_key(x);
        if (key > cand && key >= kth) above += __expf(x - mx);
      }
      above = block_sum<float>(above, redf);
      if (!(above <= budget)) t |= (1u << bit);
    }
    thr = t > kth ? t : kth;
  }
  if (out_logit_thresh && tid == 0) {
    // smallest logit (after temperature) that stays in the support, for inspection and tests
    const uint32_t u = (thr & 0x80000000u) ? (thr & 0x7fffffffu) : ~thr;
    out_logit_thresh[blockIdx.x] = __uint_as_float(u);
  }

  // inverse CDF in index order: thread t owns the contiguous chunk [t * per, (t + 1) * per)
  const int per = (V + kSampleThreads - 1) / kSampleThreads;
  const int lo = tid * per, hi = min(lo + per, V);
  float mine = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float x = load_logit(row, i, inv_temp);
    if (order_key(x) >= thr) mine += __expf(x - mx);
  }
  // exclusive scan over the 1024 chunk sums
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += n;
  }
  if ((tid & 31) == 31) scan[tid >> 5] = incl;
  if (tid == 0) s_pick = -1;
  __syncthreads();
  if (tid < 32) {
    float w = scan[tid];
    float wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, wi, o);
      if (tid >= o) wi += n;
    }
    scan[tid] = wi - w;  // exclusive prefix of the warps
    if (tid == 31) redf[0] = wi;  // total mass of the support
  }
  __syncthreads();
  const float total = redf[0];
  const float before = scan[tid >> 5] + incl - mine;
  const float target = uniform[blockIdx.x] * total;
  if (mine > 0.f && target >= before && target < before + mine) {
    float run = before;
    int pick = -1;
    for (int i = lo; i < hi; ++i) {
      const float x = load_logit(row, i, inv_temp);
      if (order_key(x) >= thr) {
        pick = i;  // last supported index of the chunk catches rounding at the upper edge
        run += __expf(x - mx);
        if (target < run) break;
      }
    }
    s_pick = pick;
  }
  __syncthreads();
  if (tid == 0) {
    int pick = s_pick;
    if (pick < 0) {
      // rounding put the target past the last chunk: fall back to the arg-max
      pick = 0;
      float best = -FLT_MAX;
      for (int i = 0; i < V; ++i) {
        const float x = load_logit(row, i, inv_temp);
        if (x > best) { best = x; pick = i; }
      }
    }
    out[blockIdx.x] = pick;
  }
}

}  // namespace
}  // namespace tpb

using namespace tpb;

extern "C" {

int tpb_embedding_fwd(const long long* ids, const void* table, void* out, long long n, int H,
                      long long V, void* stream) {
  if (n <= 0) return 0;
  if (H <= 0 || (H & 7)) return -1;
  const long long total = n * (H / 8);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  embedding_fwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, n, H, V);
  return (int)cudaGetLastError();
}

// dw is bf16 (f32 = 0) or fp32 (f32 = 1) and is accumulated into (zero it first for a fresh gradient).
int tpb_embedding_bwd(const long long* ids, const void* dy, void* dw, long long n, int H,
                      long long V, int f32, void* stream) {
  if (n <= 0) return 0;
  if (H <= 0 || (H & 1)) return -1;
  const long long total = n * (H / 2);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  auto st = static_cast<cudaStream_t>(stream);
  if (f32)
    embedding_bwd_kernel<true><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)dy, dw, n, H, V);
  else
    embedding_bwd_kernel<false><<<grid, 256, 0, st>>>(ids, (const __nv_bfloat16*)dy, dw, n, H, V);
  return (int)cudaGetLastError();
}

int tpb_kv_append(const void* src, void* dst, const int* pos, const int* block_table, int pos0,
                  int B, int T, int H, int D, int block, int max_blocks, long long s_b,
                  long long s_t, long long s_h, long long d_b, long long d_t, long long d_h,
                  void* stream) {
  if (B <= 0 || T <= 0) return 0;
  if (D <= 0 || (D & 7) || ((s_b | s_t | s_h | d_b | d_t | d_h) & 7)) return -1;
  if (block_table && (block <= 0 || max_blocks <= 0)) return -2;
  KvAppendParams p;
  p.src = (const __nv_bfloat16*)src; p.dst = (__nv_bfloat16*)dst; p.pos = pos;
  p.block_table = block_table; p.pos0 = pos0; p.B = B; p.T = T; p.H = H; p.D = D;
  p.block = block; p.max_blocks = max_blocks;
  p.s_b = s_b; p.s_t = s_t; p.s_h = s_h; p.d_b = d_b; p.d_t = d_t; p.d_h = d_h;
  const long long total = (long long)B * T * H * (D / 8);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  kv_append_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// qkv [B, Hq + 2 Hkv, D] (batch stride qkv_b); q_out [B, Hq, D] contiguous; caches addressed as
// base + b * c_b + t * c_t + h * c_h with `cap` token rows; pos int32 [B].
int tpb_decode_qkv_prep(const void* qkv, void* q_out, void* k_cache, void* v_cache, const float* cos_t,
                        const float* sin_t, const int* pos, int B, int Hq, int Hkv, int D, int cap,
                        int max_pos, long long qkv_b, long long c_b, long long c_t, long long c_h,
                        void* stream) {
  TPB_NVTX("tpb_decode_qkv_prep");
  if (B <= 0) return 0;
  if (D <= 0 || (D & 15) || ((qkv_b | c_b | c_t | c_h) & 7) || !pos) return -2;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache)) & 15)
    return -2;
  DecodeQkvParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.q_out = (__nv_bfloat16*)q_out;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.cos_t = cos_t; p.sin_t = sin_t; p.pos = pos;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.cap = cap; p.max_pos = max_pos;
  p.qkv_b = qkv_b; p.c_b = c_b; p.c_t = c_t; p.c_h = c_h;
  const long long total = (long long)B * (Hq + 2 * Hkv) * (D / 16);
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  decode_qkv_prep_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return (int)cudaGetLastError();
}

// logits [rows, V] (fp32 when f32 = 1, else bf16); uniform [rows] in [0, 1); out int64 [rows];
// thresh (optional) fp32 [rows] receives the smallest tempered logit kept in the support.
int tpb_sample(const void* logits, const float* uniform, long long* out, float* thresh, int rows,
               int V, long long row_stride, int f32, float temperature, int top_k, float top_p,
               void* stream) {
  if (rows <= 0) return 0;
  if (V <= 0 || !(temperature > 0.f)) return -1;
  auto st = static_cast<cudaStream_t>(stream);
  const float inv_t = 1.f / temperature;
  if (f32)
    sample_kernel<float><<<rows, kSampleThreads, 0, st>>>((const float*)logits, uniform, out, thresh, V,
                                                          row_stride, inv_t, top_k, top_p);
  else
    sample_kernel<__nv_bfloat16><<<rows, kSampleThreads, 0, st>>>((const __nv_bfloat16*)logits, uniform, out,
                                                                  thresh, V, row_stride, inv_t, top_k, top_p);
  return (int)cudaGetLastError();
}

}  // extern "C"
