// Persistent, warp-specialised bf16 GEMM for sm_100a:
//   C[m, n] (+)= sum_k A(m, k) * B(n, k)  (+ bias[n])
// TMA (128-byte swizzle) feeds a multi-stage shared-memory ring, one elected thread issues
// tcgen05.mma into a double-buffered TMEM accumulator, four epilogue warps drain it with
// tcgen05.ld. Each operand may be K-major (the reduce dim is contiguous) or MN-major, so the
// forward (x W^T), the input-gradient (dy W) and the weight-gradient (dy^T x) products all run
// without a transpose pass.
//
// Optional "ready flags" let the producer wait until a row block of B has landed in local
// memory; the all-gather that lands it runs in copy CTAs of the same launch (ag_gemm below).
//
// Replaces the cuBLASLt path of the reference (p10/src/backend/cuda/CudaBlasGemm.cpp:694-1052).
#include "sm100.cuh"
#include "tpb_api.h"

#include <mutex>

namespace tpb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;  // warp0 TMA, warp1 MMA, warps 2..5 epilogue
constexpr int kGroupM = 16;        // rasterisation: 16 M-tiles share a column sweep for L2 reuse

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = 2 * BLOCK_N;  // double-buffered accumulator (256 or 512)
};

struct GemmParams {
  int M, N, K;
  int ldc;
  void* C;
  const void* bias;  // bf16 or fp32 [N], may be null
  int bias_f32;
  int out_f32;      // 1: C is fp32, 0: C is bf16
  int accumulate;   // 1: C += result
  float alpha;
  uint32_t* status;
  unsigned long long wait_ns;
  // optional readiness flags for B rows (local memory, set by copy CTAs): flag[i] >= want
  // means rows [i*rows_per_flag, (i+1)*rows_per_flag) of B are valid.
  const uint32_t* b_flags;
  int rows_per_flag;
  uint32_t flag_want;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  int per_group = kGroupM * tiles_n;
  int g = tile / per_group;
  int first_m = g * kGroupM;
  int gsize = min(tiles_m - first_m, kGroupM);
  int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using Cfg = GemmCfg<BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + Cfg::kStages;
  uint64_t* tfull = bars + 2 * Cfg::kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_w = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (p.M + kBlockM - 1) / kBlockM;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kBlockK - 1) / kBlockK;

  if (threadIdx.x == 0) {
    *abort_w = 0;
    for (int i = 0; i < Cfg::kStages; ++i) {
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
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{abort_w, p.status, p.wait_ns};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        if (p.b_flags) {
          int r0 = tn * BLOCK_N;
          int r1 = min(r0 + BLOCK_N, p.N) - 1;
          for (int f = r0 / p.rows_per_flag; f <= r1 / p.rows_per_flag && ok; ++f) {
            ok = flag_wait_ge(p.b_flags + f, p.flag_want, false, p.status, p.wait_ns, 10);
            if (!ok) *abort_w = 1;
          }
          if (!ok) break;
          // rows were written with generic-proxy stores by other CTAs; order them before TMA reads
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % Cfg::kStages;
          uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, wc, 1)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sa, &tmA, &full[s], kb * kBlockK, tm * kBlockM);
          } else {
#pragma unroll
            for (int c = 0; c < kBlockM / 64; ++c)
              tma_load_2d(sa + c * (kBlockK * 128), &tmA, &full[s], tm * kBlockM + c * 64,
                          kb * kBlockK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmB, &full[s], kb * kBlockK, tn * BLOCK_N);
          } else {
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c)
              tma_load_2d(sb + c * (kBlockK * 128), &tmB, &full[s], tn * BLOCK_N + c * 64,
                          kb * kBlockK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(kBlockM, BLOCK_N, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++lt) {
        int as = lt & 1;
        uint32_t aph = (lt >> 1) & 1;
        if (!mbar_wait(&tempty[as], aph ^ 1, wc, 2)) break;
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + as * BLOCK_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          int s = it % Cfg::kStages;
          uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&full[s], ph, wc, 3)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int j = 0; j < kBlockK / kUmmaK; ++j) {
            uint64_t da = A_MN ? make_smem_desc_sw128(sa + j * 2048, kBlockK * 128, 1024)
                               : make_smem_desc_sw128(sa + j * 32, 16, 1024);
            uint64_t db = B_MN ? make_smem_desc_sw128(sb + j * 2048, kBlockK * 128, 1024)
                               : make_smem_desc_sw128(sb + j * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb | j) != 0);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[as]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++lt) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      int as = lt & 1;
      uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait_warp(&tfull[as], aph, wc, 4)) break;
      tc_fence_after_sync();
      const int row = tm * kBlockM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * BLOCK_N;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 32) {
        const int col0 = tn * BLOCK_N + c;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        if (row < p.M) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          const bool full_chunk = (col0 + 32 <= p.N);
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (full_chunk || col0 + i < p.N) {
                float b = p.bias_f32
                              ? reinterpret_cast<const float*>(p.bias)[col0 + i]
                              : __bfloat162float(
                                    reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
                v[i] += b;
              }
            }
          }
          if (p.out_f32) {
            float* crow = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (p.accumulate) {
                  float4 old = *reinterpret_cast<float4*>(crow + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) crow[i] = p.accumulate ? crow[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* crow =
                reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (p.accumulate) {
                  uint4 old = *reinterpret_cast<uint4*>(crow + i);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = __bfloat1622float2(ob[j]);
                    v[i + 2 * j] += f.x;
                    v[i + 2 * j + 1] += f.y;
                  }
                }
                uint4 o;
                __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  ob2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) {
                  float x = p.accumulate ? __bfloat162float(crow[i]) + v[i] : v[i];
                  crow[i] = __float2bfloat16(x);
                }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[as]);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_w) {
    // A wait gave up: leave time for bulk copies still in flight to land before the CTA exits.
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver call and needs a context bound to the calling thread;
// threads that have only been handed a device by the runtime (autograd workers) have none
// until their first runtime call that touches the device.
void ensure_thread_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

static EncodeTiledFn get_encode_fn() {
  ensure_thread_context();
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// 2-D bf16 tensor map with 128-byte swizzle: inner dim `d0` contiguous, outer dim `d1` with
// a stride of `ld` elements; box = {64, box1}.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t ld,
                      uint32_t box1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BLOCK_N, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                       int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BLOCK_N>;
  auto kern = gemm_bf16_kernel<BLOCK_N, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int tiles = ((p.M + kBlockM - 1) / kBlockM) * ((p.N + BLOCK_N - 1) / BLOCK_N);
  int grid = tiles < max_ctas ? tiles : max_ctas;
  if (grid <= 0) return 0;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

int gemm_bf16_dispatch(const void* A, const void* B, void* C, const void* bias, int M, int N,
                       int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                       int bias_f32, int accumulate, float alpha, const uint32_t* b_flags,
                       int rows_per_flag, uint32_t flag_want, int max_ctas, uint32_t* status,
                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  const int block_n = (N > 128) ? 256 : 128;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, K, M, lda, kBlockM);
  else r = make_tmap_2d_bf16(&ta, A, M, K, lda, kBlockK);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, K, N, ldb, block_n);
  else r = make_tmap_2d_bf16(&tb, B, N, K, ldb, kBlockK);
  if (r) return r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C; p.bias = bias; p.bias_f32 = bias_f32;
  p.out_f32 = out_f32; p.accumulate = accumulate; p.alpha = alpha; p.status = status;
  p.wait_ns = kDefaultWaitNs;
  p.b_flags = b_flags; p.rows_per_flag = rows_per_flag > 0 ? rows_per_flag : 1;
  p.flag_want = flag_want;
  if (max_ctas <= 0) max_ctas = sm_count();
#define TPB_GEMM_CASE(BN, AM, BM) \
  if (block_n == BN && (bool)a_mn == AM && (bool)b_mn == BM) \
    return launch_gemm<BN, AM, BM>(ta, tb, p, max_ctas, stream);
  TPB_GEMM_CASE(256, false, false)
  TPB_GEMM_CASE(256, false, true)
  TPB_GEMM_CASE(256, true, false)
  TPB_GEMM_CASE(256, true, true)
  TPB_GEMM_CASE(128, false, false)
  TPB_GEMM_CASE(128, false, true)
  TPB_GEMM_CASE(128, true, false)
  TPB_GEMM_CASE(128, true, true)
#undef TPB_GEMM_CASE
  return -3;
}

}  // namespace tpb

extern "C" int tpb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N,
                             int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                             int bias_f32, int accumulate, float alpha, uint32_t* status,
                             void* stream) {
  return tpb::gemm_bf16_dispatch(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32,
                                 bias_f32, accumulate, alpha, nullptr, 0, 0, 0, status,
                                 static_cast<cudaStream_t>(stream));
}
