// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a:
//   C[m, n] (+)= alpha * sum_k A(m, k) * B(n, k)  (+ bias[n])
// Two CTAs of a cluster compute one 256 x 256 tile: each owns 128 rows of A and of the
// accumulator (its own TMEM) and HALF of the B tile (128 of the 256 columns); one thread of the
// leader CTA issues every MMA for the pair and the tensor cores of both SMs read the two B halves
// from each other's shared memory. Per MMA a CTA therefore fetches 4 KB + 4 KB instead of the
// 4 KB + 8 KB of a one-CTA 128 x 256 tile, and TMA writes 32 KB per k-block instead of 48 KB: the
// shared-memory traffic that limits the one-CTA kernel drops by a third, which also buys power.
//
// Every CTA loads its own operands with TMA into its own ring (each byte is fetched once; no load
// is multicast), and both CTAs' loads count their bytes on the LEADER's `full` barrier
// (`cp.async.bulk.tensor ... .cta_group::2` lets the completion barrier live in the peer CTA), so the
// issuing thread waits on one local barrier per k-block and no thread relays anything: a relay
// thread doing one release-scoped remote arrive per k-block was measured at ~1000 cycles per
// arrive, three times the MMA time of the k-block. `tcgen05.commit` with a cluster mask frees ring
// slots and publishes finished accumulators in both CTAs at once. Every wait is bounded.
//
// The reference calls cuBLASLt here (p10/src/backend/cuda/CudaBlasGemm.cpp:694-1052).
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int kPairM = 256;   // rows of a tile (128 per CTA)
constexpr int kPairK = 64;
constexpr int kPairThreads = 192;  // warp 0 TMA, warp 1 TMEM owner + MMA issue (leader), warps 2..5 epilogue
constexpr int kPairABytes = 128 * kPairK * 2;
// BN = columns of a tile (256 or 128); each CTA stages BN / 2 of them.
template <int BN>
struct PairCfg {
  static constexpr int kHalfN = BN / 2;
  static constexpr int kBBytes = kHalfN * kPairK * 2;
  static constexpr int kStageBytes = kPairABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? 6 : 8;
  static constexpr int kSmem = kStages * kStageBytes + 1024 + 512;
};
constexpr int kPairGroupM = 8;

struct PairParams {
  int M, N, K, ldc;
  void* C;
  const void* bias;
  int bias_f32, out_f32, accumulate;
  float alpha;
  uint32_t* status;
  unsigned long long wait_ns;
  // Split of the last, partially filled wave along K (null sk_ws = off): the tiles left over after
  // the full waves are each computed by `nsplit` pairs over disjoint K ranges; helpers park fp32
  // partial tiles in sk_ws and bump sk_flags[tail tile], the owner folds them into its epilogue.
  float* sk_ws;
  uint32_t* sk_flags;
  long long* trace;  // optional [6][128] clock64 stamps of pair 0: rows 0/3 = leader/peer producer got its slot,
                     // 1 = operands of the k-block landed, 5 = its MMAs issued
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}" ::"r"(smem_u32(bar)),
      "r"(rank)
      : "memory");
}
// Shared-window address of `bar`'s twin (same offset) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
// 2-D tile load into THIS CTA's shared memory whose byte count completes on `bar_cluster`, a barrier
// of either CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* m, uint32_t bar_cluster, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(m), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_pair_f16_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                 uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All MMAs issued so far by this thread complete -> one arrival on `bar` in BOTH CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"((uint16_t)3)
      : "memory");
}

__device__ __forceinline__ void pair_stamp(const PairParams& p, int pair, int role, uint32_t it) {
  if (p.trace && pair == 0 && it < 128) p.trace[role * 128 + it] = clock64();
}

struct PairWork {
  int tile, kb0, kb1, split, nsplit, tail_idx;
};
struct PairSched {
  int npairs, full_per, tail, nsplit, k_blocks;
};
__device__ __forceinline__ PairSched pair_sched(int n_tiles, int npairs, int k_blocks, bool can_split) {
  PairSched sc;
  sc.npairs = npairs;
  sc.k_blocks = k_blocks;
  sc.full_per = n_tiles / npairs;
  sc.tail = n_tiles - sc.full_per * npairs;
  sc.nsplit = 1;
  if (can_split && sc.tail > 0) {
    int n = min(npairs / sc.tail, k_blocks / 8);
    sc.nsplit = n > 8 ? 8 : (n < 1 ? 1 : n);
  }
  return sc;
}
// The i-th unit of work of pair `pid`; false when the pair has no i-th unit.
__device__ __forceinline__ bool pair_work(const PairSched& sc, int pid, int i, PairWork& w) {
  w.kb0 = 0; w.kb1 = sc.k_blocks; w.split = 0; w.nsplit = 1; w.tail_idx = 0;
  if (i < sc.full_per) {
    w.tile = pid + i * sc.npairs;
    return true;
  }
  if (i > sc.full_per) return false;
  if (sc.nsplit > 1) {
    if (pid >= sc.tail * sc.nsplit) return false;
    w.tail_idx = pid / sc.nsplit;
    w.split = pid - w.tail_idx * sc.nsplit;
    w.nsplit = sc.nsplit;
    w.tile = sc.full_per * sc.npairs + w.tail_idx;
    const int qk = sc.k_blocks / sc.nsplit, rk = sc.k_blocks % sc.nsplit;  // every range is non-empty
    w.kb0 = w.split * qk + min(w.split, rk);
    w.kb1 = w.kb0 + qk + (w.split < rk ? 1 : 0);
    return true;
  }
  if (pid >= sc.tail) return false;
  w.tile = sc.full_per * sc.npairs + pid;
  return true;
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = kPairGroupM * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * kPairGroupM;
  const int gsize = min(tiles_m - first_m, kPairGroupM);
  const int r = tile - g * per_group;
  tm = first_m + (r % gsize);
  tn = r / gsize;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const PairParams p) {
  using Cfg = PairCfg<BN>;
  constexpr int kPairStages = Cfg::kStages;
  constexpr int kPairStageBytes = Cfg::kStageBytes;
  constexpr int kPairN = BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* full = bars;                         // leader only: both CTAs' operands landed (tx count)
  uint64_t* empty = full + kPairStages;          // ring slot consumed (commit, both CTAs)
  uint64_t* tfull = empty + kPairStages;         // accumulator complete (commit, both CTAs)
  uint64_t* tempty = tfull + 2;                  // leader only: accumulator drained by all 8 epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile uint32_t* abort_w = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t crank = cluster_ctarank();       // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int tiles_m = (p.M + kPairM - 1) / kPairM;
  const int tiles_n = (p.N + kPairN - 1) / kPairN;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kPairK - 1) / kPairK;
  const PairSched sc = pair_sched(n_tiles, npairs, k_blocks, p.sk_ws != nullptr);
  PairWork w;

  if (threadIdx.x == 0) {
    *abort_w = 0;
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&tfull[0], 1);
    mbar_init(&tfull[1], 1);
    mbar_init(&tempty[0], 8);
    mbar_init(&tempty[1], 8);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // barriers of both CTAs are initialised and both hold their TMEM before any remote signal
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{abort_w, p.status, p.wait_ns};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (every CTA, own halves)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int wi = 0; ok && pair_work(sc, pair, wi, w); ++wi) {
        int tm, tn;
        pair_tile_coords(w.tile, tiles_m, tiles_n, tm, tn);
        const int row0 = tm * kPairM + (int)crank * 128;   // my rows of A
        const int col0 = tn * kPairN + (int)crank * Cfg::kHalfN;   // my columns (rows of B)
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait_relaxed(&empty[s], ph ^ 1, wc, 1)) { ok = false; break; }
          pair_stamp(p, pair, crank ? 3 : 0, it);
          uint8_t* sa = smem + s * kPairStageBytes;
          uint8_t* sb = sa + kPairABytes;
          if (crank == 0) mbar_arrive_expect_tx(&full[s], 2 * kPairStageBytes);
          const uint32_t fb = mapa_u32(&full[s], 0);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmA, fb, kb * kPairK, row0);
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_2d_pair(sa + c * (kPairK * 128), &tmA, fb, row0 + c * 64, kb * kPairK);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmB, fb, kb * kPairK, col0);
          } else {
#pragma unroll
            for (int c = 0; c < Cfg::kHalfN / 64; ++c) tma_load_2d_pair(sb + c * (kPairK * 128), &tmB, fb, col0 + c * 64, kb * kPairK);
          }
        }
      }
      // Tail: the leader's last commits arrive on this CTA's `empty` barriers from the other SM;
      // wait for them so that none lands after this CTA has left.
      for (int i = 0; i < kPairStages && ok; ++i, ++it) {
        if (it < (uint32_t)kPairStages) continue;  // this slot was never filled
        ok = mbar_wait_relaxed(&empty[it % kPairStages], ((it / kPairStages) & 1) ^ 1, wc, 7);
      }
    }
  } else if (warp == 1) {
    if (crank == 0) {
      // ---------------------------------------------------------- leader: MMA issue for the pair
      // (warp-uniform control flow, one elected lane issues: tcgen05 operands live in uniform registers)
      constexpr uint32_t idesc = make_idesc_f16(kPairM, kPairN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem), A_MN ? kPairK * 128 : 16);
      const uint32_t b_lo0 = smem_desc_lo(smem_u32(smem + kPairABytes), B_MN ? kPairK * 128 : 16);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int wi = 0; ok && pair_work(sc, pair, wi, w); ++wi, ++lt) {
        const int as = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (!mbar_wait_warp(&tempty[as], aph ^ 1, wc, 3)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + as * kPairN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const int s = it % kPairStages;
          const uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait_warp(&full[s], ph, wc, 4)) { ok = false; break; }
          if (lane == 0) pair_stamp(p, pair, 1, it);
          tc_fence_after_sync();
          const uint32_t a_lo = a_lo0 + s * (kPairStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + s * (kPairStageBytes >> 4);
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < kPairK / 16; ++j) {
              const uint32_t ao = A_MN ? j * (2048 >> 4) : j * (32 >> 4);
              const uint32_t bo = B_MN ? j * (2048 >> 4) : j * (32 >> 4);
              umma_pair_f16_ss(d_tmem, a_lo + ao, hi, b_lo + bo, hi, idesc, ((kb - w.kb0) | j) != 0);
            }
            umma_commit_pair(&empty[s]);
            pair_stamp(p, pair, 5, it);
          }
          __syncwarp();
        }
        if (ok) {
          if (elect_one()) umma_commit_pair(&tfull[as]);
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps per CTA, own 128 rows)
    const int q = warp & 3;
    uint32_t lt = 0;
    for (int wi = 0; pair_work(sc, pair, wi, w); ++wi, ++lt) {
      int tm, tn;
      pair_tile_coords(w.tile, tiles_m, tiles_n, tm, tn);
      const int as = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait_warp(&tfull[as], aph, wc, 6)) break;
      tc_fence_after_sync();
      const int trow = (int)crank * 128 + q * 32 + lane;   // row within the tile
      const int row = tm * kPairM + trow;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * kPairN;
      float* sk_tile = nullptr;
      if (w.nsplit > 1) {
        sk_tile = p.sk_ws + ((size_t)w.tail_idx * (w.nsplit - 1)) * (size_t)(kPairM * kPairN);
        if (w.split > 0) {
          // helper: park the fp32 partial tile, free the accumulator, signal the owner
          // layout [column / 4][row][4]: the 32 lanes of a warp (32 rows) write 512 contiguous bytes
          float* dst = sk_tile + (size_t)(w.split - 1) * (kPairM * kPairN) + (size_t)trow * 4;
#pragma unroll 1
          for (int c = 0; c < kPairN; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(dst + (size_t)((c + i) >> 2) * (kPairM * 4)) = make_float4(
                  __uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          }
          tc_fence_before_sync();
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            if (crank == 0) mbar_arrive(&tempty[as]);
            else mbar_arrive_remote(&tempty[as], 0);
            red_release_gpu_add(p.sk_flags + w.tail_idx, 1u);
          }
          continue;
        }
        // owner: every helper pair (8 epilogue warps each) must have stored its partial
        bool got = true;
        if (lane == 0) got = flag_wait_ge(p.sk_flags + w.tail_idx, 8u * (w.nsplit - 1), false, p.status, p.wait_ns, 8);
        got = __all_sync(0xffffffffu, got);
        if (!got) { *abort_w = 1; break; }
      }
#pragma unroll 1
      for (int c = 0; c < kPairN; c += 32) {
        const int col0 = tn * kPairN + c;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        if (row < p.M) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (sk_tile) {
            for (int h = 0; h < w.nsplit - 1; ++h) {
              const float* src = sk_tile + (size_t)h * (kPairM * kPairN) + (size_t)trow * 4;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                const float4 t4 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)((c + i) >> 2) * (kPairM * 4)));
                v[i] += t4.x; v[i + 1] += t4.y; v[i + 2] += t4.z; v[i + 3] += t4.w;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
          const bool full_chunk = (col0 + 32 <= p.N);
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (full_chunk || col0 + i < p.N) {
                v[i] += p.bias_f32 ? reinterpret_cast<const float*>(p.bias)[col0 + i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
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
                  const float4 old = *reinterpret_cast<float4*>(crow + i);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) crow[i] = p.accumulate ? crow[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col0;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (p.accumulate) {
                  const uint4 old = *reinterpret_cast<uint4*>(crow + i);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(ob[j]);
                    v[i + 2 * j] += f.x;
                    v[i + 2 * j + 1] += f.y;
                  }
                }
                uint4 o;
                __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) ob2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) {
                  const float x = p.accumulate ? __bfloat162float(crow[i]) + v[i] : v[i];
                  crow[i] = __float2bfloat16(x);
                }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (crank == 0) mbar_arrive(&tempty[as]);
        else mbar_arrive_remote(&tempty[as], 0);
        if (sk_tile) {
          // each owner warp checks out after consuming the partials; the last of the 8 re-arms the flag
          const unsigned old = atomicAdd(p.sk_flags + w.tail_idx, 1u);
          if (old == 8u * (w.nsplit - 1) + 7u) p.sk_flags[w.tail_idx] = 0;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_w) {
    // copies or MMAs of this pair may still be in flight: give them time before memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();   // the leader's MMAs read the peer's shared memory: nobody leaves before both are done
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

static int g_last_resident_pairs = 0;
static int g_pair_block_n = 0;  // 0 = by shape
static long long* g_pair_trace = nullptr;

template <int BN, bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const PairParams& p, int max_ctas,
                       cudaStream_t stream) {
  auto kern = gemm_pair_kernel<BN, A_MN, B_MN>;
  constexpr int kPairSmem = PairCfg<BN>::kSmem;
  // The tile loop is static (tile += pairs), so every pair of the grid must be resident at once:
  // the grid is capped at the number of 2-CTA clusters that the device can hold, which is below
  // SMs / 2 when some TPCs have a single SM enabled.
  static int resident = 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = kPairSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (resident == 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
    if (e != cudaSuccess) return (int)e;
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess) return (int)e;
    if (n <= 0) return -4;
    resident = n;
  }
  g_last_resident_pairs = resident;
  const int tiles = ((p.M + kPairM - 1) / kPairM) * ((p.N + BN - 1) / BN);
  int pairs = max_ctas / 2;
  if (resident < pairs) pairs = resident;
  // fewer tiles than pairs: with a workspace the idle pairs take K ranges of those tiles
  const bool deep = (p.K + kPairK - 1) / kPairK >= 16;
  if (tiles < pairs && !(p.sk_ws && deep && tiles * 2 <= pairs)) pairs = tiles;
  if (pairs <= 0) return 0;
  cfg.gridDim = dim3(2 * pairs);
  return (int)cudaLaunchKernelEx(&cfg, kern, ta, tb, p);
}

// Same contract as gemm_bf16_dispatch for the plain product (no flags, no fused collective).
int gemm_pair_dispatch(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                       int ldb, int ldc, int a_mn, int b_mn, int out_f32, int bias_f32, int accumulate,
                       float alpha, int max_ctas, uint32_t* status, cudaStream_t stream, int block_n) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  if (max_ctas <= 0) max_ctas = sm_count();
  // Tile width: 256 columns. The 128-column form (more tiles, less quantisation loss) measured 25 %
  // slower per flop and is only taken on request (narrow outputs).
  const int bn = block_n == 128 ? 128 : 256;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, K, M, lda, 128);
  else r = make_tmap_2d_bf16(&ta, A, M, K, lda, kPairK);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, K, N, ldb, bn / 2);
  else r = make_tmap_2d_bf16(&tb, B, N, K, ldb, kPairK);
  if (r) return r;
  PairParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.C = C; p.bias = bias; p.bias_f32 = bias_f32; p.out_f32 = out_f32;
  p.accumulate = accumulate; p.alpha = alpha; p.status = status; p.wait_ns = kDefaultWaitNs;
  p.trace = g_pair_trace;
  splitk_workspace(&p.sk_ws, &p.sk_flags);
#define TPB_PAIR_CASE(BN, AM, BM) \
  if (bn == BN && (bool)a_mn == AM && (bool)b_mn == BM) return launch_pair<BN, AM, BM>(ta, tb, p, max_ctas, stream);
  TPB_PAIR_CASE(256, false, false)
  TPB_PAIR_CASE(256, false, true)
  TPB_PAIR_CASE(256, true, false)
  TPB_PAIR_CASE(256, true, true)
  TPB_PAIR_CASE(128, false, false)
  TPB_PAIR_CASE(128, false, true)
  TPB_PAIR_CASE(128, true, false)
  TPB_PAIR_CASE(128, true, true)
#undef TPB_PAIR_CASE
  return -3;
}

}  // namespace tpb

extern "C" void tpb_gemm_pair_block_n(int v) { tpb::g_pair_block_n = v; }
extern "C" void tpb_gemm_pair_trace(void* buf) { tpb::g_pair_trace = static_cast<long long*>(buf); }
// Number of CTA pairs that the last launch found resident at once (0 before the first launch).
extern "C" int tpb_gemm_pair_resident() { return tpb::g_last_resident_pairs; }

// The CTA-pair kernel through its own entry point (benchmarks, tests); tpb_gemm_bf16 picks it by shape.
extern "C" int tpb_gemm_bf16_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                  int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32, int bias_f32,
                                  int accumulate, float alpha, uint32_t* status, void* stream) {
  TPB_NVTX("tpb_gemm_bf16_pair");
  return tpb::gemm_pair_dispatch(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, bias_f32, accumulate,
                                 alpha, 0, status, static_cast<cudaStream_t>(stream), tpb::g_pair_block_n);
}
