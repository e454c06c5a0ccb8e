// Grouped (ragged) bf16 GEMM on tcgen05 for mixture-of-experts layers.
//
// Tokens are stored expert-major in one [rows, K] buffer; expert e owns rows
// [offs[e], offs[e + 1]) where every offs[e] is a multiple of 128 and the padding rows are zero
// (the dispatch kernel lays tokens out that way), so that a 128-row tile never straddles two
// experts and padded rows contribute nothing to weight gradients. Offsets live on the device:
// a tiny prep kernel turns them into a tile table, the persistent GEMM reads the tile count
// from device memory, and no host synchronisation is needed for data-dependent routing.
//
//   mode 0 (forward / input gradient): C[r, :] = A[r, :] * B[e]^T for r in expert e
//            B[e] is [N, K] (K-major) or, with b_mn, stored [K_red, N] (W[e] as [N_red, K_out]).
//   mode 1 (weight gradient): C[e] = A[rows_e, :]^T * B[rows_e, :]  ([N, K] per expert), the
//            reduction runs over the expert's rows.
//
// Replaces the reference's CUTLASS 2.x Sm80 GemmGrouped (p10/src/backend/cuda/
// GroupedGemmKernels.cu:102-235, device-built problem descriptors :102-133); the Blackwell
// kernel to beat is its compile-only CuTeDSL template
// (tensorplay/compiler/backends/stax/codegen/cutedsl/cutedsl_grouped_gemm.py).
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int kGBlockM = 128;
constexpr int kGBlockK = 64;
constexpr int kGThreads = 192;

template <int BLOCK_N>
struct GCfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kABytes = kGBlockM * kGBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kGBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
  static constexpr int kTmemCols = 2 * BLOCK_N;
};

struct GroupedParams {
  int G, N, K;          // mode 0: per-row GEMM N x K ; mode 1: output N x K per expert
  int mode;
  const int* offs;      // [G + 1] padded row offsets (device)
  const int* tile_expert;  // mode 0: [max_tiles] expert of each M tile ; built by prep kernel
  const int* tile_row;     // mode 0: [max_tiles] first row of each M tile
  const int* n_mtiles;     // device scalar: number of valid M tiles
  void* C;
  long long ldc;        // mode 0: row stride of C ; mode 1: N_out row stride inside an expert
  long long c_expert_stride;  // mode 1: elements between experts
  int out_f32, accumulate;
  uint32_t* status;
  unsigned long long wait_ns;
};

// Tile table for mode 0 (M tiles of every expert, expert-major), one thread per expert: expert e
// owns tiles [ceil(offs[e] / 128) ...) of its own row range, and because every offset is a multiple
// of 128 the experts' tile ranges are disjoint and their positions follow from the offsets alone.
__global__ void __launch_bounds__(256)
grouped_prep_kernel(const int* __restrict__ offs, int G, int* __restrict__ tile_expert,
                    int* __restrict__ tile_row, int* __restrict__ n_mtiles, int max_tiles) {
  const int base = offs[0];
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < G; e += gridDim.x * blockDim.x) {
    const int r0 = offs[e], r1 = offs[e + 1];
    int n = (r0 - base) / kGBlockM;
    for (int r = r0; r < r1 && n < max_tiles; r += kGBlockM, ++n) {
      tile_expert[n] = e;
      tile_row[n] = r;
    }
    if (e == G - 1) {
      const int total = (r1 - base) / kGBlockM;
      *n_mtiles = total < max_tiles ? total : max_tiles;
    }
  }
}

template <int BLOCK_N, bool B_MN>
__global__ void __launch_bounds__(kGThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GroupedParams p) {
  using Cfg = GCfg<BLOCK_N>;
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
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  // mode 0: tiles = M tiles x N tiles ; mode 1: tiles = G x (N/128) x (K/BLOCK_N)
  int n_tiles;
  int tiles_k_out = 0;
  if (p.mode == 0) {
    n_tiles = *p.n_mtiles * tiles_n;
  } else {
    tiles_k_out = (p.K + BLOCK_N - 1) / BLOCK_N;
    n_tiles = p.G * ((p.N + kGBlockM - 1) / kGBlockM) * tiles_k_out;
  }

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

  // tile -> coordinates
  auto decode = [&](int tile, int& e, int& row0, int& c0, int& kb0, int& kb1) {
    if (p.mode == 0) {
      // N tiles fastest so that one expert's A tile is reused from L2 across its N tiles
      const int mt = tile / tiles_n;
      e = p.tile_expert[mt];
      row0 = p.tile_row[mt];
      c0 = (tile % tiles_n) * BLOCK_N;
      kb0 = 0;
      kb1 = (p.K + kGBlockK - 1) / kGBlockK;
    } else {
      const int per_e = ((p.N + kGBlockM - 1) / kGBlockM) * tiles_k_out;
      e = tile / per_e;
      const int r = tile % per_e;
      row0 = (r / tiles_k_out) * kGBlockM;  // output row (n index)
      c0 = (r % tiles_k_out) * BLOCK_N;     // output col (k index)
      kb0 = p.offs[e] / kGBlockK;
      kb1 = p.offs[e + 1] / kGBlockK;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int e, row0, c0, kb0, kb1;
        decode(tile, e, row0, c0, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, wc, 1)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[s], Cfg::kStageBytes);
          if (p.mode == 0) {
            tma_load_2d(sa, &tmA, &full[s], kb * kGBlockK, row0);
            if (!B_MN) {
              tma_load_3d(sb, &tmB, &full[s], kb * kGBlockK, c0, e);
            } else {
#pragma unroll
              for (int c = 0; c < BLOCK_N / 64; ++c)
                tma_load_3d(sb + c * (kGBlockK * 128), &tmB, &full[s], c0 + c * 64, kb * kGBlockK, e);
            }
          } else {
            // A = dY^T: MN-major operand from dY [rows, N] ; B = X^T from X [rows, K]
#pragma unroll
            for (int c = 0; c < kGBlockM / 64; ++c)
              tma_load_2d(sa + c * (kGBlockK * 128), &tmA, &full[s], row0 + c * 64, kb * kGBlockK);
#pragma unroll
            for (int c = 0; c < BLOCK_N / 64; ++c)
              tma_load_2d(sb + c * (kGBlockK * 128), &tmB, &full[s], c0 + c * 64, kb * kGBlockK);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (p.mode == 0)
                                 ? make_idesc_f16(kGBlockM, BLOCK_N, 1, 0, B_MN ? 1 : 0)
                                 : make_idesc_f16(kGBlockM, BLOCK_N, 1, 1, 1);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int e, row0, c0, kb0, kb1;
        decode(tile, e, row0, c0, kb0, kb1);
        if (kb1 <= kb0) continue;  // expert without rows: nothing to accumulate (lt counts used tiles)
        const int as = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        ++lt;
        if (!mbar_wait(&tempty[as], aph ^ 1, wc, 2)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * BLOCK_N;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % Cfg::kStages;
          const uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&full[s], ph, wc, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
          const bool a_mn = p.mode == 1;
          const bool b_mn = p.mode == 1 || B_MN;
#pragma unroll
          for (int j = 0; j < kGBlockK / 16; ++j) {
            uint64_t da = a_mn ? make_smem_desc_sw128(sa + j * 2048, kGBlockK * 128, 1024)
                               : make_smem_desc_sw128(sa + j * 32, 16, 1024);
            uint64_t db = b_mn ? make_smem_desc_sw128(sb + j * 2048, kGBlockK * 128, 1024)
                               : make_smem_desc_sw128(sb + j * 32, 16, 1024);
            umma_f16_ss(d_tmem, da, db, idesc, (kb != kb0) || (j != 0));
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[as]);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t lt = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      int e, row0, c0, kb0, kb1;
      decode(tile, e, row0, c0, kb0, kb1);
      const int as = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      const bool empty_k = kb1 <= kb0;  // an expert without tokens: its weight gradient is zero
      if (!empty_k) ++lt;
      if (!empty_k) {
        if (!mbar_wait_warp(&tfull[as], aph, wc, 4)) break;
        tc_fence_after_sync();
      }
      const int row = row0 + q * 32 + lane;
      const int row_lim = (p.mode == 0) ? p.offs[e + 1] : p.N;
      const int col_lim = (p.mode == 0) ? p.N : p.K;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * BLOCK_N;
#pragma unroll 1
      for (int c = 0; c < BLOCK_N; c += 32) {
        const int col0 = c0 + c;
        if (col0 >= col_lim) break;
        uint32_t r[32];
        if (!empty_k) {
          tmem_ld_32x32b_x32(t_row + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        if (row < row_lim) {
          const bool full_chunk = col0 + 32 <= col_lim;
          const size_t base = (p.mode == 0) ? (size_t)row * p.ldc + col0
                                            : (size_t)e * p.c_expert_stride + (size_t)row * p.ldc + col0;
          if (p.out_f32) {
            float* crow = reinterpret_cast<float*>(p.C) + base;
            for (int i = 0; i < 32; ++i)
              if (full_chunk || col0 + i < col_lim) {
                float v = __uint_as_float(r[i]);
                crow[i] = p.accumulate ? crow[i] + v : v;
              }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + base;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[i + j]);
                if (p.accumulate) {
                  uint4 old = *reinterpret_cast<uint4*>(crow + i);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    float2 f = __bfloat1622float2(ob[j]);
                    v[2 * j] += f.x;
                    v[2 * j + 1] += f.y;
                  }
                }
                uint4 o;
                __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) ob2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                *reinterpret_cast<uint4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < col_lim) {
                  float v = __uint_as_float(r[i]);
                  if (p.accumulate) v += __bfloat162float(crow[i]);
                  crow[i] = __float2bfloat16(v);
                }
            }
          }
        }
      }
      if (!empty_k) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty[as]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_w) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BLOCK_N, bool B_MN>
static int launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, const GroupedParams& p,
                          cudaStream_t stream) {
  using Cfg = GCfg<BLOCK_N>;
  auto kern = grouped_gemm_kernel<BLOCK_N, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<sm_count(), kGThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

}  // namespace tpb

using namespace tpb;

// Workspace (ints) needed by tpb_grouped_gemm for `max_rows` rows: 2 * tiles + 1.
extern "C" int tpb_grouped_workspace_ints(int max_rows, int G) {
  return 2 * (max_rows / kGBlockM + G + 1) + 4;
}

// mode 0: C[rows, N] = A[rows, K] x B[e]^T (B: [G, N, K], or with b_mn [G, K_red, N_out] i.e. the
//         weight itself for the input gradient). mode 1: C[G, N, K] = A[rows, N]^T x B[rows, K].
// offs: device [G + 1], multiples of 128; rows beyond offs[G] are ignored; max_rows bounds offs[G].
extern "C" int tpb_grouped_gemm(const void* A, const void* B, void* C, const int* offs, int G,
                                int max_rows, int N, int K, int mode, int b_mn, int out_f32,
                                int accumulate, int* workspace, uint32_t* status, void* stream_) {
  TPB_NVTX("tpb_grouped_gemm");
  cudaStream_t stream = (cudaStream_t)stream_;
  if (G <= 0 || max_rows <= 0) return 0;
  if (N % 8 || K % 8 || max_rows % kGBlockM) return -2;
  GroupedParams p;
  p.G = G; p.N = N; p.K = K; p.mode = mode; p.offs = offs; p.C = C;
  p.out_f32 = out_f32; p.accumulate = accumulate; p.status = status; p.wait_ns = kDefaultWaitNs;
  const int max_tiles = max_rows / kGBlockM + G + 1;
  int* tile_expert = workspace;
  int* tile_row = workspace + max_tiles;
  int* n_mtiles = workspace + 2 * max_tiles;
  p.tile_expert = tile_expert; p.tile_row = tile_row; p.n_mtiles = n_mtiles;
  CUtensorMap ta, tb;
  int r;
  if (mode == 0) {
    grouped_prep_kernel<<<(G + 255) / 256, 256, 0, stream>>>(offs, G, tile_expert, tile_row, n_mtiles, max_tiles);
    p.ldc = N; p.c_expert_stride = 0;
    const int block_n = N > 128 ? 256 : 128;
    if ((r = make_tmap_2d_bf16(&ta, A, K, max_rows, K, kGBlockM))) return r;
    if (!b_mn) {
      uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)G};
      uint64_t str[3] = {1, (uint64_t)K, (uint64_t)N * K};
      uint32_t box[3] = {64, (uint32_t)block_n, 1};
      if ((r = make_tmap_bf16(&tb, B, 3, dims, str, box, 1))) return r;
      return block_n == 256 ? launch_grouped<256, false>(ta, tb, p, stream)
                            : launch_grouped<128, false>(ta, tb, p, stream);
    }
    // B stored [G, K_red, N_out]: inner dim = N_out
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)K, (uint64_t)G};
    uint64_t str[3] = {1, (uint64_t)N, (uint64_t)N * K};
    uint32_t box[3] = {64, 64, 1};
    if ((r = make_tmap_bf16(&tb, B, 3, dims, str, box, 1))) return r;
    return block_n == 256 ? launch_grouped<256, true>(ta, tb, p, stream)
                          : launch_grouped<128, true>(ta, tb, p, stream);
  }
  // mode 1: A = dY [rows, N] (MN-major), B = X [rows, K] (MN-major); C[e] is [N, K]
  p.ldc = K; p.c_expert_stride = (long long)N * K;
  const int block_n = K > 128 ? 256 : 128;
  if ((r = make_tmap_2d_bf16(&ta, A, N, max_rows, N, kGBlockK))) return r;
  if ((r = make_tmap_2d_bf16(&tb, B, K, max_rows, K, kGBlockK))) return r;
  return block_n == 256 ? launch_grouped<256, true>(ta, tb, p, stream)
                        : launch_grouped<128, true>(ta, tb, p, stream);
}
