// Quantized linear algebra for inference on sm_100a.
//
//   * int8 x int8 -> int32 GEMM on the tcgen05 tensor cores (kind::i8) with a fused
//     row-scale x column-scale (+ bias) epilogue that emits bf16 (A8W8, rowwise scales);
//   * weight-only GEMV for decode (W8A16 per-channel, W4A16 group-wise): weights are read
//     once at their packed width, activations stay in bf16, accumulation in fp32;
//   * quantise / dequantise kernels (rowwise int8, int8/int4 weights -> bf16, fp8 e4m3 / e5m2).
//
// Capability reference: p10/src/backend/cuda/QuantGemmKernels.cu:92-1611 (weight-only and A8W8
// GEMMs), IntMM.cu:62 (int8 matmul), AffineQuantKernels.cu:1302 (fp8 quantise / dequantise).
#include <cuda_fp8.h>

#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {
namespace {

constexpr int kQThreads = 192;
constexpr int kQBlockM = 128;
constexpr int kQBlockN = 256;
constexpr int kQBlockK = 128;  // int8 elements = one 128-byte swizzle row
constexpr int kQStages = 4;
constexpr int kQABytes = kQBlockM * kQBlockK;
constexpr int kQBBytes = kQBlockN * kQBlockK;
constexpr int kQStageBytes = kQABytes + kQBBytes;
constexpr int kQSmem = kQStages * kQStageBytes + 256 + 1024;

struct I8Params {
  int M, N, K, ldc;
  __nv_bfloat16* C;
  const float* a_scale;  // [M] or null
  const float* b_scale;  // [N] or null
  const __nv_bfloat16* bias;  // [N] or null
  uint32_t* status;
  unsigned long long wait_ns;
};

// Persistent kernel: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue.
__global__ void __launch_bounds__(kQThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const I8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kQStages * kQStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kQStages;
  uint64_t* tfull = empty + kQStages;   // 2
  uint64_t* tempty = tfull + 2;         // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_w = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kQBlockM - 1) / kQBlockM;
  const int tiles_n = (p.N + kQBlockN - 1) / kQBlockN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kQBlockK - 1) / kQBlockK;

  if (threadIdx.x == 0) {
    *abort_w = 0;
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 4);
    mbar_init(&tempty[1], 4);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{abort_w, p.status, p.wait_ns};

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        // column-major over tiles: consecutive CTAs share the B (weight) tile row in L2
        const int tm = tile % tiles_m, tn = tile / tiles_m;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kQStages;
          const uint32_t ph = (it / kQStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, wc, 1)) { ok = false; break; }
          uint8_t* sa = smem + s * kQStageBytes;
          mbar_arrive_expect_tx(&full[s], kQStageBytes);
          tma_load_2d(sa, &tmA, &full[s], kb * kQBlockK, tm * kQBlockM);
          tma_load_2d(sa + kQABytes, &tmB, &full[s], kb * kQBlockK, tn * kQBlockN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_i8(kQBlockM, kQBlockN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
        const int as = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (!mbar_wait(&tempty[as], aph ^ 1, wc, 2)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * kQBlockN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kQStages;
          const uint32_t ph = (it / kQStages) & 1;
          if (!mbar_wait(&full[s], ph, wc, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * kQStageBytes);
          const uint32_t sb = sa + kQABytes;
#pragma unroll
          for (int j = 0; j < kQBlockK / 32; ++j)  // one kind::i8 instruction covers K = 32
            umma_i8_ss(d_tmem, make_smem_desc_sw128(sa + j * 32, 16, 1024),
                       make_smem_desc_sw128(sb + j * 32, 16, 1024), idesc, (kb | j) != 0);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[as]);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
      const int tm = tile % tiles_m, tn = tile / tiles_m;
      const int as = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait_warp(&tfull[as], aph, wc, 4)) break;
      tc_fence_after_sync();
      const int row = tm * kQBlockM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * kQBlockN;
      const float sa = (p.a_scale && row < p.M) ? p.a_scale[row] : 1.f;
#pragma unroll 1
      for (int c = 0; c < kQBlockN; c += 32) {
        const int col0 = tn * kQBlockN + c;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        if (row < p.M) {
          __nv_bfloat16* dst = p.C + (size_t)row * p.ldc + col0;
          const bool full_chunk = (col0 + 32 <= p.N) && ((p.ldc & 7) == 0);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = min(col0 + i, p.N - 1);
            float x = (float)(int)r[i] * sa * (p.b_scale ? __ldg(p.b_scale + col) : 1.f);
            if (p.bias) x += __bfloat162float(p.bias[col]);
            v[i] = x;
          }
          if (full_chunk) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(v[g * 8 + 0], v[g * 8 + 1]);
              __nv_bfloat162 t1 = __floats2bfloat162_rn(v[g * 8 + 2], v[g * 8 + 3]);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(v[g * 8 + 4], v[g * 8 + 5]);
              __nv_bfloat162 t3 = __floats2bfloat162_rn(v[g * 8 + 6], v[g * 8 + 7]);
              o.x = *reinterpret_cast<uint32_t*>(&t0);
              o.y = *reinterpret_cast<uint32_t*>(&t1);
              o.z = *reinterpret_cast<uint32_t*>(&t2);
              o.w = *reinterpret_cast<uint32_t*>(&t3);
              *reinterpret_cast<uint4*>(dst + g * 8) = o;
            }
          } else {
            for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = __float2bfloat16(v[i]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[as]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ weight-only GEMV (decode)
// y[m, n] = sum_k x[m, k] * dq(W[n, k]) for up to 8 rows of x. A warp owns kCols output columns at a
// time; every lane owns 16 consecutive k per step: it unpacks the 8 x 16 activations of its slice to
// fp32 registers once and reuses them for all kCols columns, so the kernel streams the packed weights
// once and the activations (L2-resident) only 1/kCols times per column. Integer codes become fp32
// by placing them in the mantissa of 2^23 (one permute + one add, no conversion instruction) and
// the inner products use packed fp32x2 FMAs.
constexpr int kGemvCols = 4;

__device__ __forceinline__ float code_to_f32(uint32_t byte_in_low_bits) {
  // 0x4B000000 = 2^23; the code sits in the low mantissa bits
  return __uint_as_float(0x4B000000u | byte_in_low_bits) - 8388608.f;
}

template <int BITS>
__global__ void __launch_bounds__(256)
wq_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
               const __nv_bfloat16* __restrict__ scale, const __nv_bfloat16* __restrict__ zero,
               const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N,
               int K, int group, long long ldx, long long ldy) {
  constexpr int kRows = 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups_per_row = (group > 0) ? K / group : 1;
  const int n_groups = (N + kGemvCols - 1) / kGemvCols;
  for (int ng = blockIdx.x * 8 + warp; ng < n_groups; ng += gridDim.x * 8) {
    const int n0 = ng * kGemvCols;
    float2 acc[kGemvCols][kRows / 2];  // acc[c][r / 2].{x, y} = rows r, r + 1
#pragma unroll
    for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
      for (int r = 0; r < kRows / 2; ++r) acc[c][r] = make_float2(0.f, 0.f);
    // the packed weights of step i + 1 are requested before the arithmetic of step i: the HBM
    // latency of the only stream that comes from DRAM hides behind the FMAs
    auto load_w = [&](int k0, uint32_t (&dst)[kGemvCols][4]) {
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) {
        const int n = min(n0 + c, N - 1);
        if (k0 >= K) {
          dst[c][0] = dst[c][1] = dst[c][2] = dst[c][3] = 0;
        } else if (BITS == 8) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(w + (size_t)n * K + k0));
          dst[c][0] = v.x; dst[c][1] = v.y; dst[c][2] = v.z; dst[c][3] = v.w;
        } else {
          const uint2 v = __ldg(reinterpret_cast<const uint2*>(w + (size_t)n * (K / 2) + k0 / 2));
          dst[c][0] = v.x; dst[c][1] = v.y; dst[c][2] = 0; dst[c][3] = 0;
        }
      }
    };
    uint32_t wq[kGemvCols][4], wn[kGemvCols][4];
    load_w(lane * 16, wq);
    for (int k0 = lane * 16; k0 < K; k0 += 32 * 16) {
      load_w(k0 + 32 * 16, wn);
      // activations of this k slice: xr[j][r / 2] = (x[r][k0 + j], x[r + 1][k0 + j])
      float2 xr[16][kRows / 2];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        if (r < M) {
          const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)r * ldx + k0);
          lo = __ldg(xp);
          hi = __ldg(xp + 1);
        }
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const uint32_t u = words[j >> 1];
          const float f = __uint_as_float((j & 1) ? (u & 0xffff0000u) : (u << 16));
          if (r & 1) xr[j][r >> 1].y = f; else xr[j][r >> 1].x = f;
        }
      }
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) {
        float sc = 1.f, zp = 0.f;
        if (group > 0 || BITS == 4) {
          // group-wise: the slice of 16 k lies inside one group (group % 16 == 0)
          const int n = min(n0 + c, N - 1);
          const int g = group > 0 ? k0 / group : 0;
          sc = __bfloat162float(scale[(size_t)n * groups_per_row + g]);
          if (BITS == 4) zp = zero ? __bfloat162float(zero[(size_t)n * groups_per_row + g]) : 8.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float wv;
          if (BITS == 8) {
            // signed byte -> biased code (b ^ 0x80) in [0, 255], value = code - 128
            const uint32_t code = ((wq[c][j >> 2] >> ((j & 3) * 8)) & 0xffu) ^ 0x80u;
            wv = code_to_f32(code) - 128.f;
          } else {
            const uint32_t code = (wq[c][j >> 3] >> ((j & 7) * 4)) & 0xfu;
            wv = code_to_f32(code) - zp;
          }
          if (group > 0 || BITS == 4) wv *= sc;
          const float2 w2 = make_float2(wv, wv);
#pragma unroll
          for (int r = 0; r < kRows / 2; ++r) acc[c][r] = __ffma2_rn(xr[j][r], w2, acc[c][r]);
        }
      }
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) wq[c][i] = wn[c][i];
    }
#pragma unroll
    for (int c = 0; c < kGemvCols; ++c) {
      const int n = n0 + c;
      float sc = 1.f;
      if (group <= 0 && BITS == 8 && n < N) sc = __bfloat162float(scale[n]);  // per-channel scale applied once
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        float a = (r & 1) ? acc[c][r >> 1].y : acc[c][r >> 1].x;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && r < M && n < N) {
          a *= sc;
          if (bias) a += __bfloat162float(bias[n]);
          y[(size_t)r * ldy + n] = __float2bfloat16(a);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ weight-only GEMV on the warp MMA
// Same contract as wq_gemv_kernel, for K that is a multiple of the chunk (64 k for 8-bit, 128 k
// for 4-bit). With at most 8 rows of x the op is bound by streaming the packed weights, and the
// CUDA-core version spends 8 FMAs per weight; here the weights of 16 output columns form the
// 16 x 16 A tile of mma.sync.m16n8k16 and the (up to) 8 rows of x its 16 x 8 B tile, so a weight
// costs only its dequantisation (3-5 instructions). tcgen05 needs the operands in shared memory
// and a 64/128-row accumulator in TMEM: for an 8-row product the warp-level MMA, fed straight from
// the registers the weights were loaded into, is the shorter path. The sum over k is order-free, so
// lane (g, t) takes 16 consecutive bytes of weight rows g and g + 8 (16 or 32 k) and the matching
// k of x row g: every global load is a full 16-byte vector and no shuffles are needed.
// A CTA owns TILES x 16 output columns; its 8 warps split K and reduce through shared memory.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Stages of the per-warp weight ring. The kernel is bound by bytes in flight, not by arithmetic:
// at ~2 us of loaded HBM latency an SM needs ~90 KB outstanding to draw its share of the
// bandwidth, far more than a register double buffer holds, so the packed weights go through
// cp.async into a shared-memory ring that is STAGES - 1 chunks ahead of the arithmetic. Every lane
// reads back exactly the 16-byte pieces it requested itself, so the ring needs no barrier.
template <int TILES>
struct GemvRing {
  static constexpr int kStages = TILES == 1 ? 6 : 4;
  static constexpr int kStageVecs = 2 * TILES * 32;  // uint4 per stage per warp
  static constexpr int kBytes = 8 * kStages * kStageVecs * 16;
};

template <int BITS, int TILES, int KS>
__global__ void __launch_bounds__(256)
wq_gemv_mma_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
                   const __nv_bfloat16* __restrict__ scale, const __nv_bfloat16* __restrict__ zero,
                   const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N,
                   int K, int group, long long ldx, long long ldy) {
  constexpr int KL = BITS == 8 ? 16 : 32;  // k per lane per chunk = 16 bytes of packed weights
  constexpr int CH = 4 * KL;
  constexpr int S = GemvRing<TILES>::kStages;
  constexpr int SV = GemvRing<TILES>::kStageVecs;
  constexpr bool kScaled = BITS == 4;      // 8-bit: grouped scales are a run-time property
  extern __shared__ uint4 gemv_ring[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  uint4* my_ring = gemv_ring + (size_t)warp * S * SV;
  // KS warps split K for one row tile (TILES x 16 columns); the CTA covers 8 / KS row tiles
  const int kw = warp % KS;
  const int n_base = (blockIdx.x * (8 / KS) + warp / KS) * TILES * 16;
  const int n_chunks = K / CH;
  const int gpr = group > 0 ? K / group : 1;
  const bool grouped = kScaled || group > 0;
  const size_t row_bytes = BITS == 8 ? (size_t)K : (size_t)K / 2;
  int rown[TILES][2];
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int h = 0; h < 2; ++h) rown[tl][h] = min(n_base + tl * 16 + g + 8 * h, N - 1);
  float acc[TILES][4];
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[tl][i] = 0.f;

  // one commit group per chunk, also when the chunk does not exist: the group count stays uniform
  auto issue_w = [&](int c, int stage) {
    if (c < n_chunks) {
      const size_t off = (size_t)(c * CH + t * KL) * BITS / 8;
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int h = 0; h < 2; ++h)
          cp_async_16(my_ring + (size_t)stage * SV + (tl * 2 + h) * 32 + lane,
                      w + (size_t)rown[tl][h] * row_bytes + off);
    }
    cp_async_commit();
  };
  // x rows of a chunk (KL bf16 of row g, zeros past M) and the chunk's group scales are requested
  // one chunk ahead in registers: they come from L1 / L2
  auto load_x = [&](int c, uint32_t (&dst)[KL / 2]) {
    if (g < M && c < n_chunks) {
      const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)g * ldx + c * CH + t * KL);
#pragma unroll
      for (int i = 0; i < KL / 8; ++i) {
        const uint4 v = __ldg(xp + i);
        dst[4 * i + 0] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < KL / 2; ++i) dst[i] = 0u;
    }
  };
  auto load_s = [&](int c, float (&sc)[TILES][2], float (&zp)[TILES][2]) {
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sc[tl][h] = 1.f;
        zp[tl][h] = 8.f;
        if (grouped && c < n_chunks) {
          const size_t idx = (size_t)rown[tl][h] * gpr + (group > 0 ? (c * CH + t * KL) / group : 0);
          sc[tl][h] = __bfloat162float(scale[idx]);
          if (BITS == 4 && zero) zp[tl][h] = __bfloat162float(zero[idx]);
        }
      }
  };

#pragma unroll
  for (int s = 0; s < S - 1; ++s) issue_w(kw + KS * s, s);
  uint32_t xw[KL / 2], xn[KL / 2];
  float scw[TILES][2], zpw[TILES][2], scn[TILES][2], zpn[TILES][2];
  load_x(kw, xw);
  load_s(kw, scw, zpw);
  int it = 0;
  for (int c = kw; c < n_chunks; c += KS, ++it) {
    issue_w(c + KS * (S - 1), (it + S - 1) % S);
    load_x(c + KS, xn);
    load_s(c + KS, scn, zpn);
    cp_async_wait<S - 1>();  // this chunk's group has landed (S - 1 younger ones may be pending)
    const uint4* st = my_ring + (size_t)(it % S) * SV;
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl) {
      const uint4 w0 = st[(tl * 2 + 0) * 32 + lane], w1 = st[(tl * 2 + 1) * 32 + lane];
      const uint32_t wv[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
      float sc[2], zs[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // 4-bit: the nibble goes to the top mantissa bits of 1.0 (v = 1 + code / 16) and one FMA
        // gives (code - zp) * sc = v * (16 sc) - (16 + zp) * sc, the constant exact to 2^-24 of 16 sc
        sc[h] = BITS == 4 ? 16.f * scw[tl][h] : scw[tl][h];
        zs[h] = -(16.f + zpw[tl][h]) * scw[tl][h];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (BITS == 8) {
          uint32_t a[2][2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t q = wv[h][i] ^ 0x80808080u;  // signed byte -> biased code, value = code - 128
            float f[4];
            f[0] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7440)) - 8388736.f;
            f[1] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7441)) - 8388736.f;
            f[2] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7442)) - 8388736.f;
            f[3] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7443)) - 8388736.f;
            if (group > 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) f[j] *= sc[h];
            }
            a[h][0] = pack_bf16x2(f[0], f[1]);
            a[h][1] = pack_bf16x2(f[2], f[3]);
          }
          mma_bf16_16816(acc[tl], a[0][0], a[1][0], a[0][1], a[1][1], xw[2 * i], xw[2 * i + 1]);
        } else {
          uint32_t a[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t q = wv[h][i];
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t sh = (4 * j <= 19) ? (q << (19 - 4 * j)) : (q >> (4 * j - 19));
              f[j] = fmaf(__uint_as_float((sh & 0x00780000u) | 0x3F800000u), sc[h], zs[h]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) a[h][j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
          }
          mma_bf16_16816(acc[tl], a[0][0], a[1][0], a[0][1], a[1][1], xw[4 * i], xw[4 * i + 1]);
          mma_bf16_16816(acc[tl], a[0][2], a[1][2], a[0][3], a[1][3], xw[4 * i + 2], xw[4 * i + 3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < KL / 2; ++i) xw[i] = xn[i];
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        scw[tl][h] = scn[tl][h];
        zpw[tl][h] = zpn[tl][h];
      }
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the reduction buffer reuses the memory
  float* red = reinterpret_cast<float*>(gemv_ring);  // [8][TILES * 128]
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp * (TILES * 128) + tl * 128 + lane * 4 + i] = acc[tl][i];
  __syncthreads();
  for (int o = threadIdx.x; o < (8 / KS) * TILES * 128; o += 256) {
    const int rt = o / (TILES * 128), e = o % (TILES * 128);  // row tile of the CTA, element in it
    float a = 0.f;
#pragma unroll
    for (int wi = 0; wi < KS; ++wi) a += red[(rt * KS + wi) * (TILES * 128) + e];
    // accumulator element (lane l, register ci) = (column g + 8 * (ci / 2), row 2 t + (ci & 1))
    const int tl = e >> 7, l = (e >> 2) & 31, ci = e & 3;
    const int n = (blockIdx.x * (8 / KS) + rt) * TILES * 16 + tl * 16 + (l >> 2) + ((ci & 2) ? 8 : 0);
    const int r = 2 * (l & 3) + (ci & 1);
    if (n < N && r < M) {
      if (group <= 0 && BITS == 8) a *= __bfloat162float(scale[n]);  // per-channel scale applied once
      if (bias) a += __bfloat162float(bias[n]);
      y[(size_t)r * ldy + n] = __float2bfloat16(a);
    }
  }
}

// Second version of the warp-MMA GEMV: the default (tpb_wq_gemv_config(tiles, 3) selects the first one
// for comparison). It passes the same numerics tests and measures 0.054 against 0.063 ms (8 bits) and
// 0.074 against 0.090 ms (4 bits, group 128) on 8 x 28672 x 8192.
// GROUPED: scales (and, for 4 bits, zero points) per group of 2^gshift k; otherwise (8 bits only)
// one scale per output column, applied once at the end. The loop is written for instruction count
// (a profile showed ~70 % issue-slot utilisation with "not selected" as the top stall, i.e. the
// kernel is issue-bound, not memory-bound): pointers advance by constants, the group index is a
// shift, the ring stage is a counter, and the x / scale registers ping-pong through two bodies.
// FOLD (4 bits, groups of at least one chunk = 128 k): the nibbles enter the MMA as the bf16 numbers
// 128 + code, two per LOP3 - nibbles j and j + 4 of a word share a register, and the x registers are
// permuted to the same pairing once per chunk - and scale and zero point are applied to the chunk's
// partial sum instead of to every weight: acc += s * (sum (128 + code) x - (128 + zp) * sum x), the sum
// of x coming from one more MMA per k-step against a row of ones. 0.9 instead of 3.5 ALU instructions
// per weight; the fp32 partial sums keep the cancellation of the 128 exact to about 2^-14 of a code.
template <int BITS, int TILES, int KS, bool GROUPED, bool FOLD = false>
__global__ void __launch_bounds__(256)
wq_gemv_mma_v2_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
                   const __nv_bfloat16* __restrict__ scale, const __nv_bfloat16* __restrict__ zero,
                   const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int M, int N,
                   int K, int gshift, long long ldx, long long ldy) {
  static_assert(BITS == 8 || GROUPED, "4-bit weights are group-quantised");
  constexpr int KL = BITS == 8 ? 16 : 32;  // k per lane per chunk = 16 bytes of packed weights
  constexpr int CH = 4 * KL;
  constexpr int S = GemvRing<TILES>::kStages;
  constexpr int SV = GemvRing<TILES>::kStageVecs;
  constexpr int kStepBytes = KS * CH * BITS / 8;  // distance between a warp's consecutive chunks
  extern __shared__ uint4 gemv_ring[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  uint4* my_ring = gemv_ring + (size_t)warp * S * SV + lane;
  // KS warps split K for one row tile (TILES x 16 columns); the CTA covers 8 / KS row tiles
  const int kw = warp % KS;
  const int n_base = (blockIdx.x * (8 / KS) + warp / KS) * TILES * 16;
  const int n_chunks = K / CH;
  const int gpr = GROUPED ? (K >> gshift) : 1;
  const size_t row_bytes = BITS == 8 ? (size_t)K : (size_t)K / 2;
  const uint8_t* wptr[TILES][2];   // next chunk to request, per weight row of this lane
  size_t srow[TILES][2];           // row offset into the scale / zero tables
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = min(n_base + tl * 16 + g + 8 * h, N - 1);
      wptr[tl][h] = w + (size_t)n * row_bytes + (size_t)(kw * CH + t * KL) * BITS / 8;
      srow[tl][h] = (size_t)n * gpr;
    }
  float acc[TILES][4];
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[tl][i] = 0.f;

  int c_issue = kw, st_issue = 0;
  // one commit group per chunk, also when the chunk does not exist: the group count stays uniform
  auto issue_w = [&]() {
    if (c_issue < n_chunks) {
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          cp_async_16(my_ring + st_issue * SV + (tl * 2 + h) * 32, wptr[tl][h]);
          wptr[tl][h] += kStepBytes;
        }
    }
    cp_async_commit();
    c_issue += KS;
    st_issue = st_issue + 1 == S ? 0 : st_issue + 1;
  };
  const bool x_row = g < M;
  const uint4* xptr = reinterpret_cast<const uint4*>(x + (size_t)(x_row ? g : 0) * ldx + kw * CH + t * KL);
  // x rows of a chunk (KL bf16 of row g, zeros past M) and the chunk's group scales are requested
  // one chunk ahead in registers: they come from L1 / L2
  auto load_x = [&](int c, uint32_t (&dst)[KL / 2]) {
    if (x_row && c < n_chunks) {
#pragma unroll
      for (int i = 0; i < KL / 8; ++i) {
        const uint4 v = __ldg(xptr + i);
        dst[4 * i + 0] = v.x; dst[4 * i + 1] = v.y; dst[4 * i + 2] = v.z; dst[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < KL / 2; ++i) dst[i] = 0u;
    }
    xptr += KS * CH / 8;
  };
  auto load_s = [&](int c, float (&sc)[TILES][2], float (&zs)[TILES][2]) {
    if (!GROUPED) return;
    const int gi = (c * CH + t * KL) >> gshift;
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float s = 1.f, z = 8.f;
        if (c < n_chunks) {
          s = __bfloat162float(scale[srow[tl][h] + gi]);
          if (BITS == 4 && zero) z = __bfloat162float(zero[srow[tl][h] + gi]);
        }
        // 4-bit: the nibble goes to the top mantissa bits of 1.0 (v = 1 + code / 16) and one FMA
        // gives (code - zp) * s = v * (16 s) - (16 + zp) * s, the constant exact to 2^-24 of 16 s
        if (FOLD) {
          sc[tl][h] = s;
          zs[tl][h] = -(128.f + z);
        } else {
          sc[tl][h] = BITS == 4 ? 16.f * s : s;
          zs[tl][h] = -(16.f + z) * s;
        }
      }
  };

  int st_use = 0;
  // arithmetic of one chunk, with the registers that hold its x rows and scales
  auto compute = [&](const uint32_t (&xw)[KL / 2], const float (&sc)[TILES][2], const float (&zs)[TILES][2]) {
    cp_async_wait<S - 1>();  // this chunk's group has landed (S - 1 younger ones may be pending)
    const uint4* st = my_ring + st_use * SV;
    st_use = st_use + 1 == S ? 0 : st_use + 1;
    if constexpr (FOLD) {
      // x pairs (k, k + 4) of every run of 8 k, and the chunk's sum of x per column (rows all equal)
      uint32_t px[KL / 2];
#pragma unroll
      for (int i = 0; i < KL / 8; ++i) {
        px[4 * i + 0] = __byte_perm(xw[4 * i + 0], xw[4 * i + 2], 0x5410);
        px[4 * i + 1] = __byte_perm(xw[4 * i + 0], xw[4 * i + 2], 0x7632);
        px[4 * i + 2] = __byte_perm(xw[4 * i + 1], xw[4 * i + 3], 0x5410);
        px[4 * i + 3] = __byte_perm(xw[4 * i + 1], xw[4 * i + 3], 0x7632);
      }
      float xs[4] = {0.f, 0.f, 0.f, 0.f};
      constexpr uint32_t kOnes = 0x3F803F80u;
#pragma unroll
      for (int i = 0; i < KL / 4; ++i) mma_bf16_16816(xs, kOnes, kOnes, kOnes, kOnes, px[2 * i], px[2 * i + 1]);
#pragma unroll
      for (int tl = 0; tl < TILES; ++tl) {
        const uint4 w0 = st[(tl * 2 + 0) * 32], w1 = st[(tl * 2 + 1) * 32];
        const uint32_t wv[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t a[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 4; ++j) a[h][j] = ((wv[h][i] >> (4 * j)) & 0x000F000Fu) | 0x43004300u;
          mma_bf16_16816(tmp, a[0][0], a[1][0], a[0][1], a[1][1], px[4 * i], px[4 * i + 1]);
          mma_bf16_16816(tmp, a[0][2], a[1][2], a[0][3], a[1][3], px[4 * i + 2], px[4 * i + 3]);
        }
        // accumulator element ci: weight row g + 8 (ci / 2), x row 2 t + (ci & 1)
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
          acc[tl][ci] = fmaf(sc[tl][ci >> 1], fmaf(zs[tl][ci >> 1], xs[ci], tmp[ci]), acc[tl][ci]);
      }
      return;
    }
#pragma unroll
    for (int tl = 0; tl < TILES; ++tl) {
      const uint4 w0 = st[(tl * 2 + 0) * 32], w1 = st[(tl * 2 + 1) * 32];
      const uint32_t wv[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (BITS == 8) {
          uint32_t a[2][2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t q = wv[h][i] ^ 0x80808080u;  // signed byte -> biased code, value = code - 128
            float f[4];
            f[0] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7440)) - 8388736.f;
            f[1] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7441)) - 8388736.f;
            f[2] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7442)) - 8388736.f;
            f[3] = __uint_as_float(__byte_perm(q, 0x4B000000u, 0x7443)) - 8388736.f;
            if (GROUPED) {
#pragma unroll
              for (int j = 0; j < 4; ++j) f[j] *= sc[tl][h];
            }
            a[h][0] = pack_bf16x2(f[0], f[1]);
            a[h][1] = pack_bf16x2(f[2], f[3]);
          }
          mma_bf16_16816(acc[tl], a[0][0], a[1][0], a[0][1], a[1][1], xw[2 * i], xw[2 * i + 1]);
        } else {
          uint32_t a[2][4];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t q = wv[h][i];
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t sh = (4 * j <= 19) ? (q << (19 - 4 * j)) : (q >> (4 * j - 19));
              f[j] = fmaf(__uint_as_float((sh & 0x00780000u) | 0x3F800000u), sc[tl][h], zs[tl][h]);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) a[h][j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
          }
          mma_bf16_16816(acc[tl], a[0][0], a[1][0], a[0][1], a[1][1], xw[4 * i], xw[4 * i + 1]);
          mma_bf16_16816(acc[tl], a[0][2], a[1][2], a[0][3], a[1][3], xw[4 * i + 2], xw[4 * i + 3]);
        }
      }
    }
  };

#pragma unroll
  for (int s = 0; s < S - 1; ++s) issue_w();
  uint32_t xa[KL / 2], xb[KL / 2];
  float sa[TILES][2], za[TILES][2], sb[TILES][2], zb[TILES][2];
  load_x(kw, xa);
  load_s(kw, sa, za);
  for (int c = kw; c < n_chunks; c += 2 * KS) {
    issue_w();
    load_x(c + KS, xb);
    load_s(c + KS, sb, zb);
    compute(xa, sa, za);
    if (c + KS >= n_chunks) break;
    issue_w();
    load_x(c + 2 * KS, xa);
    load_s(c + 2 * KS, sa, za);
    compute(xb, sb, zb);
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the reduction buffer reuses the memory
  float* red = reinterpret_cast<float*>(gemv_ring);  // [8][TILES * 128]
#pragma unroll
  for (int tl = 0; tl < TILES; ++tl)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp * (TILES * 128) + tl * 128 + lane * 4 + i] = acc[tl][i];
  __syncthreads();
  for (int o = threadIdx.x; o < (8 / KS) * TILES * 128; o += 256) {
    const int rt = o / (TILES * 128), e = o % (TILES * 128);  // row tile of the CTA, element in it
    float a = 0.f;
#pragma unroll
    for (int wi = 0; wi < KS; ++wi) a += red[(rt * KS + wi) * (TILES * 128) + e];
    // accumulator element (lane l, register ci) = (column g + 8 * (ci / 2), row 2 t + (ci & 1))
    const int tl = e >> 7, l = (e >> 2) & 31, ci = e & 3;
    const int n = (blockIdx.x * (8 / KS) + rt) * TILES * 16 + tl * 16 + (l >> 2) + ((ci & 2) ? 8 : 0);
    const int r = 2 * (l & 3) + (ci & 1);
    if (n < N && r < M) {
      if (!GROUPED) a *= __bfloat162float(scale[n]);  // per-channel scale applied once
      if (bias) a += __bfloat162float(bias[n]);
      y[(size_t)r * ldy + n] = __float2bfloat16(a);
    }
  }
}

// ------------------------------------------------------------------ quantise / dequantise
// Rowwise symmetric int8: scale = absmax / 127 per row; one CTA per row.
__global__ void __launch_bounds__(256)
quant_i8_rowwise_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                        float* __restrict__ scale, int K, long long ldx) {
  __shared__ float red[8];
  const int row = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  float mx = 0.f;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + k);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  const float s = mx > 0.f ? mx / 127.f : 1.f;
  const float inv = 1.f / s;
  if (threadIdx.x == 0) scale[row] = s;
  for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + k);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t o[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(h[j]);
      const int a = max(-127, min(127, __float2int_rn(f.x * inv)));
      const int b = max(-127, min(127, __float2int_rn(f.y * inv)));
      o[j >> 1] |= ((uint32_t)(a & 0xff) << ((j & 1) * 16)) | ((uint32_t)(b & 0xff) << ((j & 1) * 16 + 8));
    }
    *reinterpret_cast<uint2*>(q + (size_t)row * K + k) = make_uint2(o[0], o[1]);
  }
}

// Packed weights -> bf16 (prefill path: dequantise once, then the bf16 tensor-core GEMM).
template <int BITS>
__global__ void __launch_bounds__(256)
dequant_w_kernel(const uint8_t* __restrict__ w, const __nv_bfloat16* __restrict__ scale,
                 const __nv_bfloat16* __restrict__ zero, __nv_bfloat16* __restrict__ out, int N,
                 int K, int group) {
  const long long idx = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;  // 8 weights per thread
  if (idx >= (long long)N * K) return;
  const int n = (int)(idx / K), k = (int)(idx % K);
  const int gpr = group > 0 ? K / group : 1;
  const int g = group > 0 ? k / group : 0;
  const float s = __bfloat162float(scale[(size_t)n * gpr + g]);
  float v[8];
  if (BITS == 8) {
    const uint2 pk = *reinterpret_cast<const uint2*>(w + idx);
    const uint32_t words[2] = {pk.x, pk.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (float)(int8_t)((words[i >> 2] >> ((i & 3) * 8)) & 0xff) * s;
  } else {
    const uint32_t pk = *reinterpret_cast<const uint32_t*>(w + idx / 2);
    const float z = zero ? __bfloat162float(zero[(size_t)n * gpr + g]) : 8.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = ((float)((pk >> (i * 4)) & 0xf) - z) * s;
  }
  uint4 o;
  __nv_bfloat162 t0 = __floats2bfloat162_rn(v[0], v[1]), t1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 t2 = __floats2bfloat162_rn(v[4], v[5]), t3 = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
  o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
  *reinterpret_cast<uint4*>(out + idx) = o;
}

// fp8 quantise: q = saturate(x / scale); scale is per tensor (rows_per_scale = 0) or per row.
template <typename F8>
__global__ void __launch_bounds__(256)
fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                 uint8_t* __restrict__ q, long long n, int row_len, int per_row) {
  const long long idx = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
  if (idx >= n) return;
  const float inv = 1.f / scale[per_row ? idx / row_len : 0];
  const uint4 v = *reinterpret_cast<const uint4*>(x + idx);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  uint8_t o[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    F8 a(f.x * inv), b(f.y * inv);  // the constructor saturates to the finite range
    o[2 * j] = *reinterpret_cast<uint8_t*>(&a);
    o[2 * j + 1] = *reinterpret_cast<uint8_t*>(&b);
  }
  *reinterpret_cast<uint2*>(q + idx) = *reinterpret_cast<uint2*>(o);
}

template <typename F8>
__global__ void __launch_bounds__(256)
fp8_dequant_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                   __nv_bfloat16* __restrict__ out, long long n, int row_len, int per_row) {
  const long long idx = ((long long)blockIdx.x * 256 + threadIdx.x) * 8;
  if (idx >= n) return;
  const float s = scale[per_row ? idx / row_len : 0];
  const uint2 pk = *reinterpret_cast<const uint2*>(q + idx);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&pk);
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    F8 t;
    *reinterpret_cast<uint8_t*>(&t) = b[i];
    v[i] = (float)t * s;
  }
  uint4 o;
  __nv_bfloat162 t0 = __floats2bfloat162_rn(v[0], v[1]), t1 = __floats2bfloat162_rn(v[2], v[3]);
  __nv_bfloat162 t2 = __floats2bfloat162_rn(v[4], v[5]), t3 = __floats2bfloat162_rn(v[6], v[7]);
  o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
  o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
  *reinterpret_cast<uint4*>(out + idx) = o;
}

}  // namespace
}  // namespace tpb

using namespace tpb;

extern "C" {

// C[M, N] (bf16) = (A_q[M, K] . B_q[N, K]^T) * a_scale[m] * b_scale[n] (+ bias[n]); int8 operands,
// K a multiple of 16 and both row pitches multiples of 16 bytes (TMA).
int tpb_gemm_i8(const void* A, const void* B, void* C, const float* a_scale, const float* b_scale,
                const void* bias, int M, int N, int K, int lda, int ldb, int ldc, uint32_t* status,
                void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K & 15) || (lda & 15) || (ldb & 15)) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15) return -3;
  CUtensorMap ta, tb;
  int r = make_tmap_2d_u8(&ta, A, K, M, lda, kQBlockM);
  if (r) return r;
  r = make_tmap_2d_u8(&tb, B, K, N, ldb, kQBlockN);
  if (r) return r;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kQSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  I8Params p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.a_scale = a_scale; p.b_scale = b_scale;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = status; p.wait_ns = kDefaultWaitNs;
  const int tiles = ((M + kQBlockM - 1) / kQBlockM) * ((N + kQBlockN - 1) / kQBlockN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  gemm_i8_kernel<<<grid, kQThreads, kQSmem, static_cast<cudaStream_t>(stream)>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

static int g_gemv_tiles = 0;       // 0: pick by N; 1 / 2: 16-column tiles per CTA of the MMA kernel
static int g_gemv_force_simt = 0;  // 0 / 2: second MMA version (default); 1: always the CUDA-core kernel; 3: first MMA version; 4: second version with per-weight scaling for 4 bits too
// Tuning / comparison knobs of the weight-only GEMV (process-wide).
int tpb_wq_gemv_config(int tiles, int force_simt) {
  g_gemv_tiles = (tiles == 1 || tiles == 2) ? tiles : 0;
  g_gemv_force_simt = (force_simt >= 1 && force_simt <= 4) ? force_simt : 0;
  return 0;
}

// bits = 8: W int8 [N, K], scale bf16 [N, K/group] (group = 0: one scale per row).
// bits = 4: W uint8 [N, K/2] (two codes per byte, low nibble first), group-wise (group % 16 == 0).
int tpb_wq_gemv(const void* x, const void* w, const void* scale, const void* zero, const void* bias,
                void* y, int M, int N, int K, int bits, int group, long long ldx, long long ldy,
                void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (bits != 8 && bits != 4) return -2;
  if (K % 16 || (ldx & 7)) return -3;
  if (group > 0 && (K % group || group % 16)) return -4;
  if (bits == 4 && group <= 0) return -4;
  auto st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16 *sc = (const __nv_bfloat16*)scale, *zp = (const __nv_bfloat16*)zero,
                      *bs = (const __nv_bfloat16*)bias;
  const int chunk = bits == 8 ? 64 : 128;
  const bool mma_ok = g_gemv_force_simt != 1 && K % chunk == 0 && (group <= 0 || group % (chunk / 4) == 0) &&
                      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  // two 16-column tiles per warp halve the reads of x, which load the L1 data path more than the weights do
  // (every lane re-reads its x slice for each weight tile: 2 KB of x against 1 KB of 4-bit weights per chunk
  // with one tile); one tile keeps more CTAs in flight when N is short. The first kernel version was slower
  // with two tiles (registers) and keeps its old rule.
  const bool second_version = g_gemv_force_simt == 0 || g_gemv_force_simt == 2 || g_gemv_force_simt == 4;
  const int tiles = g_gemv_tiles ? g_gemv_tiles
                                 : ((N + 31) / 32 >= sm_count() * (second_version ? 2 : 8) ? 2 : 1);
  const int n_groups = (N + kGemvCols - 1) / kGemvCols;
  int grid = (n_groups + 7) / 8;
  const int cap = sm_count() * 4;
  if (grid > cap) grid = cap;
  for (int m0 = 0; m0 < M; m0 += 8) {  // 8 rows of x per launch
    const __nv_bfloat16* xs = (const __nv_bfloat16*)x + (size_t)m0 * ldx;
    __nv_bfloat16* ys = (__nv_bfloat16*)y + (size_t)m0 * ldy;
    const int rows = M - m0 < 8 ? M - m0 : 8;
    const uint8_t* wp = (const uint8_t*)w;
    if (mma_ok) {
      // int4 has half the chunks of int8 for the same K: four warps per row tile keep the loop long
      const int ks = bits == 8 ? 8 : 4;
      const int per_cta = 16 * tiles * (8 / ks);
      const int g2 = (N + per_cta - 1) / per_cta;
      if (g_gemv_force_simt != 3 && (group <= 0 || (group & (group - 1)) == 0)) {
        int gshift = 0;
        while (group > 0 && (1 << gshift) < group) ++gshift;
        auto launch = [&](auto kern, int smem, int variant) {
          static bool opted_in[8] = {false, false, false, false, false, false, false, false};  // per kernel variant
          if (!opted_in[variant]) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            opted_in[variant] = true;
          }
          kern<<<g2, 256, smem, st>>>(xs, wp, sc, zp, bs, ys, rows, N, K, gshift, ldx, ldy);
        };
        if (bits == 8 && group <= 0) {
          if (tiles == 2) launch(wq_gemv_mma_v2_kernel<8, 2, 8, false>, GemvRing<2>::kBytes, 0);
          else launch(wq_gemv_mma_v2_kernel<8, 1, 8, false>, GemvRing<1>::kBytes, 1);
        } else if (bits == 8) {
          if (tiles == 2) launch(wq_gemv_mma_v2_kernel<8, 2, 8, true>, GemvRing<2>::kBytes, 2);
          else launch(wq_gemv_mma_v2_kernel<8, 1, 8, true>, GemvRing<1>::kBytes, 3);
        } else {
          // groups of at least one 128-k chunk: scale and zero point applied per chunk, not per weight
          const bool fold = gshift >= 7 && g_gemv_force_simt != 4;
          if (fold && tiles == 2) launch(wq_gemv_mma_v2_kernel<4, 2, 4, true, true>, GemvRing<2>::kBytes, 6);
          else if (fold) launch(wq_gemv_mma_v2_kernel<4, 1, 4, true, true>, GemvRing<1>::kBytes, 7);
          else if (tiles == 2) launch(wq_gemv_mma_v2_kernel<4, 2, 4, true>, GemvRing<2>::kBytes, 4);
          else launch(wq_gemv_mma_v2_kernel<4, 1, 4, true>, GemvRing<1>::kBytes, 5);
        }
        continue;
      }
      auto launch = [&](auto kern, int smem) {
        static bool opted_in[4] = {false, false, false, false};  // per kernel variant
        bool& done = opted_in[(bits == 8 ? 0 : 2) + (tiles == 2 ? 1 : 0)];
        if (!done) {
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
          done = true;
        }
        kern<<<g2, 256, smem, st>>>(xs, wp, sc, zp, bs, ys, rows, N, K, group, ldx, ldy);
      };
      if (bits == 8 && tiles == 2)
        launch(wq_gemv_mma_kernel<8, 2, 8>, GemvRing<2>::kBytes);
      else if (bits == 8)
        launch(wq_gemv_mma_kernel<8, 1, 8>, GemvRing<1>::kBytes);
      else if (tiles == 2)
        launch(wq_gemv_mma_kernel<4, 2, 4>, GemvRing<2>::kBytes);
      else
        launch(wq_gemv_mma_kernel<4, 1, 4>, GemvRing<1>::kBytes);
    } else if (bits == 8) {
      wq_gemv_kernel<8><<<grid, 256, 0, st>>>(xs, wp, sc, zp, bs, ys, rows, N, K, group, ldx, ldy);
    } else {
      wq_gemv_kernel<4><<<grid, 256, 0, st>>>(xs, wp, sc, zp, bs, ys, rows, N, K, group, ldx, ldy);
    }
  }
  return (int)cudaGetLastError();
}

int tpb_quant_i8_rowwise(const void* x, void* q, float* scale, int M, int K, long long ldx,
                         void* stream) {
  if (M <= 0 || K <= 0 || (K & 7) || (ldx & 7)) return -1;
  quant_i8_rowwise_kernel<<<M, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16*)x, (int8_t*)q, scale, K, ldx);
  return (int)cudaGetLastError();
}

int tpb_dequant_weight(const void* w, const void* scale, const void* zero, void* out, int N, int K,
                       int bits, int group, void* stream) {
  if (N <= 0 || K <= 0 || (K & 7)) return -1;
  if (group > 0 && (K % group || (group & 7))) return -2;
  const long long n = (long long)N * K;
  const int grid = (int)((n / 8 + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
  if (bits == 8)
    dequant_w_kernel<8><<<grid, 256, 0, st>>>((const uint8_t*)w, (const __nv_bfloat16*)scale,
                                              (const __nv_bfloat16*)zero, (__nv_bfloat16*)out, N, K, group);
  else if (bits == 4)
    dequant_w_kernel<4><<<grid, 256, 0, st>>>((const uint8_t*)w, (const __nv_bfloat16*)scale,
                                              (const __nv_bfloat16*)zero, (__nv_bfloat16*)out, N, K, group);
  else
    return -3;
  return (int)cudaGetLastError();
}

// fmt 0 = e4m3, 1 = e5m2; n a multiple of 8; per_row: one scale per `row_len` elements.
int tpb_fp8_quant(const void* x, const float* scale, void* q, long long n, int row_len, int per_row,
                  int fmt, void* stream) {
  if (n <= 0 || (n & 7) || (per_row && (row_len <= 0 || (row_len & 7)))) return -1;
  const int grid = (int)((n / 8 + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
  if (fmt == 0)
    fp8_quant_kernel<__nv_fp8_e4m3><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, scale, (uint8_t*)q, n, row_len, per_row);
  else
    fp8_quant_kernel<__nv_fp8_e5m2><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, scale, (uint8_t*)q, n, row_len, per_row);
  return (int)cudaGetLastError();
}

int tpb_fp8_dequant(const void* q, const float* scale, void* out, long long n, int row_len,
                    int per_row, int fmt, void* stream) {
  if (n <= 0 || (n & 7) || (per_row && (row_len <= 0 || (row_len & 7)))) return -1;
  const int grid = (int)((n / 8 + 255) / 256);
  auto st = static_cast<cudaStream_t>(stream);
  if (fmt == 0)
    fp8_dequant_kernel<__nv_fp8_e4m3><<<grid, 256, 0, st>>>((const uint8_t*)q, scale, (__nv_bfloat16*)out, n, row_len, per_row);
  else
    fp8_dequant_kernel<__nv_fp8_e5m2><<<grid, 256, 0, st>>>((const uint8_t*)q, scale, (__nv_bfloat16*)out, n, row_len, per_row);
  return (int)cudaGetLastError();
}

}  // extern "C"
