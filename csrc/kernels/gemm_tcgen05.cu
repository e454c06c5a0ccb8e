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
#include <string.h>

namespace tpb {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;  // warp0 TMA, warp1 MMA, warps 2..5 epilogue
constexpr int kGroupM = 16;        // rasterisation: 16 M-tiles share a column sweep for L2 reuse

// One unit of work of a CTA: a whole tile, or one K range of a tile of the split last wave.
// Ways in which each of the `tail` tiles of the last, partially filled wave is split along K over
// `nctas` CTAs (1 = not split). A split costs about five L2 round trips (partial store, fence, flag,
// wait, partial loads), as much as some sixteen k-blocks of MMAs: below that saving it does not pay.
// The host (grid size, tile width) and the kernel's schedule both call this.
__host__ __device__ inline int tail_nsplit(int tail, int nctas, int k_blocks) {
  int ns = nctas / tail;
  if (ns > k_blocks / 4) ns = k_blocks / 4;
  if (ns > 32) ns = 32;
  if (ns < 2) return 1;
  if (k_blocks - (k_blocks + ns - 1) / ns < 16) return 1;
  return ns;
}

struct WorkItem {
  int tile, kb0, kb1, split, nsplit, tail_idx;
};

template <int BLOCK_N>
struct GemmCfg {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : 6;
  static constexpr int kABytes = kBlockM * kBlockK * 2;
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // staging of the reduce-scatter epilogue: per epilogue warp 32 rows x 64 bf16 columns, rows padded
  // to 144 bytes (conflict-free 16-byte accesses both ways)
  static constexpr int kOutStageOff = kStages * kStageBytes + 256;
  static constexpr int kOutStageBytes = 4 * 32 * 144;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/ + kOutStageBytes;
  static constexpr int kTmemCols = 2 * BLOCK_N;  // double-buffered accumulator (256 or 512)
};

struct GemmParams {
  int M, N, K;
  // Rows of A that one TMA box brings (128, or 64 when the whole product has at most 64 rows: the MMA
  // still multiplies 128 rows, the upper 64 being whatever the stage held before - their results land in
  // accumulator rows that no epilogue reads - but each SM fills 8 KB less shared memory per k-block).
  int a_box_rows;
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
  // ---- split-K of the last, partially filled wave: when the tiles left over after the full
  // waves would occupy only a fraction of the CTAs, each of them is computed by `nsplit` CTAs over
  // disjoint K ranges; the helpers store fp32 partials to `sk_ws` and bump `sk_flags[tail tile]`,
  // the owner adds them in its epilogue (and resets the flag). Null sk_ws disables it.
  float* sk_ws;
  uint32_t* sk_flags;
  // ---- fused all-gather of one operand (ag_operand: 0 none, 1 = A rows, 2 = B rows). The
  // first n_copy blocks of the grid are copy CTAs: they pull the peers' row shards into the
  // local gathered buffer chunk by chunk and publish one flag per chunk; the GEMM producer
  // waits for the flags of the rows a tile needs (own-rank rows need no wait).
  int n_copy, ag_operand;
  int world, rank;
  const char* ag_src[16];   // ag_src[r]: rank r's shard inside rank r's gathered buffer
  char* ag_dst;             // local gathered buffer
  unsigned long long ag_shard_bytes, ag_chunk_bytes;
  int ag_rows_per_rank, ag_rows_per_flag;
  uint32_t* ag_flags;       // local, one per chunk of every rank's shard
  uint32_t* pad_local;      // signal pad: [ready_slot + r] = rank r's shard is valid at epoch
  uint32_t* pad_peer[16];
  int ready_slot, done_slot;
  uint32_t epoch;
  // When set, the epoch of this launch is *epoch_dev + 1, read on the device: the launch then
  // carries no host-side counter and can be replayed from a CUDA graph (a one-thread kernel bumps
  // the word after the launch).
  const uint32_t* epoch_dev;
  uint32_t rs_per_call;     // arrivals per launch and source (rs_expect = epoch * rs_per_call)
  int tile_m_shift;         // rotate M tiles so that locally available rows are computed first
  int tile_n_shift;         // the same along N (gathered B operand)
  // ---- fused reduce-scatter epilogue (rs_mode = 1): row block d of the product belongs to
  // rank d; tiles are stored (bf16) into rank d's staging slice [rank][rows_per_rank, N] and a
  // per-source counter on rank d is bumped; after its tiles every CTA helps reducing the slices
  // that arrived for this rank into rs_out.
  int rs_mode, rs_rows_per_rank;
  char* rs_stage[16];       // staging buffer base on every rank
  uint32_t* rs_cnt[16];     // counters on every rank ([src] = tile-quarters received from src)
  uint32_t rs_expect;       // counter value that means "all tiles of this launch arrived"
  __nv_bfloat16* rs_out;    // local [rows_per_rank, N]
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


__device__ __forceinline__ uint4 ld_peer_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t fused_epoch(const GemmParams& p) {
  return p.epoch_dev ? *reinterpret_cast<const volatile uint32_t*>(p.epoch_dev) + 1u : p.epoch;
}
__device__ __forceinline__ uint32_t fused_rs_expect(const GemmParams& p) {
  return p.epoch_dev ? fused_epoch(p) * p.rs_per_call : p.rs_expect;
}

// Copy CTAs of the fused all-gather: chunk c of peer (rank + 1 + c / chunks_per_rank).
// One thread per copy CTA drives bulk asynchronous copies through the CTA's shared memory: peer
// memory -> shared (cp.async.bulk with an mbarrier, no multicast) -> local memory (cp.async.bulk
// store), 16 KB pieces, 6 loads in flight in an 8-slot ring. A copy CTA so keeps 96 KB in flight
// instead of the 24 KB that its 192 threads reach with 8 x 16-byte loads each, which at NVLink's
// latency is the difference between 0.15 and 0.6 TB/s for 16 copy CTAs.
constexpr int kAgPiece = 16384;
constexpr int kAgSlots = 8;
constexpr int kAgDepth = 6;

__device__ __forceinline__ void bulk_store_1d(void* dst, const void* src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
}

__device__ void ag_copy_role(const GemmParams& p, uint8_t* smem, uint64_t* bars, volatile uint32_t* abort_w) {
  // publish "my shard is valid" to every peer, once
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.pad_peer[threadIdx.x] + p.ready_slot + p.rank, fused_epoch(p));
  }
  if (threadIdx.x != 0) return;
  *abort_w = 0;
  for (int i = 0; i < kAgSlots; ++i) mbar_init(&bars[i], 1);
  fence_barrier_init();
  WaitCtx wc{abort_w, p.status, p.wait_ns};
  const int cpr = (int)((p.ag_shard_bytes + p.ag_chunk_bytes - 1) / p.ag_chunk_bytes);
  const int total = cpr * (p.world - 1);
  uint32_t n_loaded = 0, n_stored = 0;
  bool ok = true;
  for (int c = blockIdx.x; c < total && ok; c += p.n_copy) {
    const int pr = c / cpr, ci = c % cpr;
    const int r = (p.rank + 1 + pr) % p.world;
    if (!flag_wait_ge(p.pad_local + p.ready_slot + r, fused_epoch(p), true, p.status, p.wait_ns, 11)) { ok = false; break; }
    const unsigned long long off = (unsigned long long)ci * p.ag_chunk_bytes;
    const unsigned long long nbytes = min(p.ag_chunk_bytes, p.ag_shard_bytes - off);
    const char* src = p.ag_src[r] + off;
    char* dst = p.ag_dst + (unsigned long long)r * p.ag_shard_bytes + off;
    const int pieces = (int)((nbytes + kAgPiece - 1) / kAgPiece);
    for (int i = 0; i < pieces + kAgDepth && ok; ++i) {
      if (i < pieces) {
        const int slot = n_loaded % kAgSlots;
        // the store that last read this slot (kAgSlots pieces ago) must be done with it
        if (n_loaded >= (uint32_t)kAgSlots) tma_store_wait_read<kAgSlots - kAgDepth - 1>();
        const uint32_t bytes = (uint32_t)min((unsigned long long)kAgPiece, nbytes - (unsigned long long)i * kAgPiece);
        mbar_arrive_expect_tx(&bars[slot], bytes);
        bulk_load_1d(smem + slot * kAgPiece, src + (size_t)i * kAgPiece, bytes, &bars[slot]);
        ++n_loaded;
      }
      if (i >= kAgDepth) {
        const int jp = i - kAgDepth;
        const int slot = n_stored % kAgSlots;
        if (!mbar_wait(&bars[slot], (n_stored / kAgSlots) & 1, wc, 13)) { ok = false; break; }
        const uint32_t bytes = (uint32_t)min((unsigned long long)kAgPiece, nbytes - (unsigned long long)jp * kAgPiece);
        bulk_store_1d(dst + (size_t)jp * kAgPiece, smem + slot * kAgPiece, bytes);
        tma_store_commit();
        ++n_stored;
      }
    }
    if (!ok) break;
    tma_store_wait_all<0>();   // the chunk is in local memory
    __threadfence();
    st_release_gpu(p.ag_flags + (size_t)r * cpr + ci, fused_epoch(p));
  }
  if (!ok) {
    // loads of this thread may still be in flight into shared memory: give them time before the CTA leaves
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tma_store_wait_all<0>();
  // the sources may overwrite their shards once every reader is done
  __threadfence_system();
  unsigned prev = atomicAdd(p.ag_flags + (size_t)p.world * cpr, 1u);
  if (prev == (unsigned)p.n_copy - 1) {
    p.ag_flags[(size_t)p.world * cpr] = 0;
    for (int r = 0; r < p.world; ++r) st_release_sys(p.pad_peer[r] + p.done_slot + p.rank, fused_epoch(p));
  }
}

// Wait until rows [r0, r1) of the gathered operand are in local memory.
__device__ __forceinline__ bool ag_wait_rows(const GemmParams& p, int r0, int r1) {
  const int cpr = (int)((p.ag_shard_bytes + p.ag_chunk_bytes - 1) / p.ag_chunk_bytes);
  bool waited = false;
  for (int row = r0; row < r1;) {
    const int owner = row / p.ag_rows_per_rank;
    const int in_shard = row - owner * p.ag_rows_per_rank;
    const int ci = in_shard / p.ag_rows_per_flag;
    const int next = owner * p.ag_rows_per_rank + min((ci + 1) * p.ag_rows_per_flag, p.ag_rows_per_rank);
    if (owner != p.rank && owner < p.world) {
      if (!flag_wait_ge(p.ag_flags + (size_t)owner * cpr + ci, fused_epoch(p), false, p.status, p.wait_ns, 12))
        return false;
      waited = true;
    }
    row = next;
  }
  if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// After its tiles, every GEMM CTA helps summing the staged partials that arrived for this
// rank: out[i] = sum_src stage[src][i] (fp32 accumulate, rank order).
__device__ void rs_reduce_role(const GemmParams& p, int bid, int nctas, int t, const WaitCtx& wc) {
  // wait for every source's tiles (each tile bumps the counter once per epilogue warp)
  if (t < p.world &&
      !flag_wait_ge(p.rs_cnt[p.rank] + t, fused_rs_expect(p), true, p.status, p.wait_ns, 13))
    *wc.abort_smem = 1;
  // named barrier over the 128 epilogue threads (each of the four warps gets here exactly once)
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (*wc.abort_smem) return;
  const size_t per_src = (size_t)p.rs_rows_per_rank * p.N;
  const size_t nvec = per_src / 8;
  const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(p.rs_stage[p.rank]);
  // kU vectors per thread and pass, all sources' loads issued before the first use: with only 128
  // threads per CTA the memory system needs this many requests in flight to run near its bandwidth
  constexpr int kU = 4;
  const size_t stride = (size_t)nctas * 128;
  for (size_t i0 = (size_t)bid * 128 + t; i0 < nvec; i0 += stride * kU) {
    float acc[kU][8];
#pragma unroll
    for (int u = 0; u < kU; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[u][j] = 0.f;
    for (int r = 0; r < p.world; r += 2) {
      uint4 raw[2][kU];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const size_t i = i0 + (size_t)u * stride;
          raw[rr][u] = (r + rr < p.world && i < nvec)
                           ? ld_peer_v4(reinterpret_cast<const uint4*>(stage + (size_t)(r + rr) * per_src) + i)
                           : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
      for (int rr = 0; rr < 2; ++rr)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&raw[rr][u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(hb[j]);
            acc[u][2 * j] += f.x;
            acc[u][2 * j + 1] += f.y;
          }
        }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < nvec) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(acc[u][2 * j], acc[u][2 * j + 1]);
        reinterpret_cast<uint4*>(p.rs_out)[i] = o;
      }
    }
  }
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
  if ((int)blockIdx.x < p.n_copy) {
    ag_copy_role(p, smem, bars, abort_w);
    return;
  }
  const int bid = blockIdx.x - p.n_copy;
  const int nctas = gridDim.x - p.n_copy;
  const int tiles_m = (p.M + kBlockM - 1) / kBlockM;
  const int tiles_n = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (p.K + kBlockK - 1) / kBlockK;
  // schedule: full waves of whole tiles, then the tail tiles split along K over the idle CTAs
  const int full_per_cta = n_tiles / nctas;
  const int tail = n_tiles - full_per_cta * nctas;
  const int nsplit = (p.sk_ws && tail > 0) ? tail_nsplit(tail, nctas, k_blocks) : 1;
  const int n_units = tail * nsplit;
  const int n_items = full_per_cta + ((nsplit > 1 ? bid < n_units : bid < tail) ? 1 : 0);
  auto get_work = [&](int i) {
    WorkItem w;
    if (i < full_per_cta) {
      w.tile = bid + i * nctas; w.kb0 = 0; w.kb1 = k_blocks; w.split = 0; w.nsplit = 1; w.tail_idx = 0;
    } else if (nsplit > 1) {
      w.tail_idx = bid / nsplit;
      w.split = bid % nsplit;
      w.nsplit = nsplit;
      w.tile = full_per_cta * nctas + w.tail_idx;
      const int qk = k_blocks / nsplit, rk = k_blocks % nsplit;  // every range is non-empty
      w.kb0 = w.split * qk + min(w.split, rk);
      w.kb1 = w.kb0 + qk + (w.split < rk ? 1 : 0);
    } else {
      w.tile = full_per_cta * nctas + bid; w.kb0 = 0; w.kb1 = k_blocks; w.split = 0; w.nsplit = 1; w.tail_idx = 0;
    }
    return w;
  };

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
      for (int wi = 0; wi < n_items && ok; ++wi) {
        const WorkItem w = get_work(wi);
        const int tile = w.tile;
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        tm = (tm + p.tile_m_shift) % tiles_m;
      tn = (tn + p.tile_n_shift) % tiles_n;
        tn = (tn + p.tile_n_shift) % tiles_n;
        if (p.ag_operand) {
          ok = ag_wait_rows(p, p.ag_operand == 1 ? tm * kBlockM : tn * BLOCK_N,
                            p.ag_operand == 1 ? min(tm * kBlockM + kBlockM, p.M) : min(tn * BLOCK_N + BLOCK_N, p.N));
          if (!ok) { *abort_w = 1; break; }
        }
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
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          int s = it % Cfg::kStages;
          uint32_t ph = (it / Cfg::kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, wc, 1)) { ok = false; break; }
          uint8_t* sa = smem + s * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_arrive_expect_tx(&full[s], A_MN ? Cfg::kStageBytes : p.a_box_rows * (kBlockK * 2) + Cfg::kBBytes);
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
      for (int wi = 0; wi < n_items && ok; ++wi, ++lt) {
        const WorkItem w = get_work(wi);
        int as = lt & 1;
        uint32_t aph = (lt >> 1) & 1;
        if (!mbar_wait(&tempty[as], aph ^ 1, wc, 2)) break;
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + as * BLOCK_N;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
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
            umma_f16_ss(d_tmem, da, db, idesc, (kb != w.kb0) || (j != 0));
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[as]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* out_stage = smem + Cfg::kOutStageOff + q * (32 * 144);
    const bool rs_coalesce = p.rs_mode && (p.N % 64 == 0);
    uint32_t lt = 0;
    for (int wi = 0; wi < n_items; ++wi, ++lt) {
      const WorkItem w = get_work(wi);
      const int tile = w.tile;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      tm = (tm + p.tile_m_shift) % tiles_m;
      tn = (tn + p.tile_n_shift) % tiles_n;
      int as = lt & 1;
      uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait_warp(&tfull[as], aph, wc, 4)) break;
      tc_fence_after_sync();
      const int row = tm * kBlockM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + as * BLOCK_N;
      // split last wave, plain epilogue: EVERY split parks its fp32 partial rows in the workspace, then
      // each split sums a column slice of the tile over all partials and stores it: the reduction is
      // spread over the nsplit CTAs instead of queued on one owner
      if (w.nsplit > 1 && !p.rs_mode) {
        const int valid_rows = min(kBlockM, p.M - tm * kBlockM);
        float* tile_ws = p.sk_ws + (size_t)w.tail_idx * w.nsplit * (size_t)(kBlockM * BLOCK_N);
        if (q * 32 < valid_rows) {  // warp-uniform: row blocks past M are never read
          // layout [column / 4][row][4]: the 32 lanes of a warp (32 rows) write 512 contiguous bytes
          float* dst = tile_ws + (size_t)w.split * (kBlockM * BLOCK_N) + (size_t)(q * 32 + lane) * 4;
#pragma unroll 1
          for (int c = 0; c < BLOCK_N; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              __stcg(reinterpret_cast<float4*>(dst + (size_t)((c + i) >> 2) * (kBlockM * 4)),
                     make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                 __uint_as_float(r[i + 3])));
          }
        }
        tc_fence_before_sync();
        __threadfence();
        __syncwarp();
        bool got = true;
        if (lane == 0) {
          mbar_arrive(&tempty[as]);
          red_release_gpu_add(p.sk_flags + w.tail_idx, 1u);
          got = flag_wait_ge(p.sk_flags + w.tail_idx, 4u * w.nsplit, false, p.status, p.wait_ns, 14);
        }
        got = __all_sync(0xffffffffu, got);
        if (!got) { *abort_w = 1; break; }
        constexpr int kGroups = BLOCK_N / 4;
        const int g0 = w.split * kGroups / w.nsplit, g1 = (w.split + 1) * kGroups / w.nsplit;
        // Work unit of the reduction: one column group (4 columns) x one block of 32 rows, a row per
        // lane, so that a warp reads 512 contiguous bytes of every partial. The partials sit in L2
        // (written by other SMs) and every load is a full L2 round trip: eight splits of two units are
        // in flight per lane before anything is added.
        const int row_blocks = (valid_rows + 31) / 32;
        const int units = (g1 - g0) * row_blocks;
        const size_t part_stride = (size_t)(kBlockM * BLOCK_N);
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        auto finish = [&](int u, float4 acc) {
          const int g = g0 + u / row_blocks, r = (u % row_blocks) * 32 + lane;
          if (r >= valid_rows) return;
          float v[4] = {acc.x * p.alpha, acc.y * p.alpha, acc.z * p.alpha, acc.w * p.alpha};
          const int col = tn * BLOCK_N + g * 4;
          if (col >= p.N) return;
          const size_t off = (size_t)(tm * kBlockM + r) * p.ldc + col;
          const bool whole = col + 4 <= p.N;
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (whole || col + i < p.N)
                v[i] += p.bias_f32 ? reinterpret_cast<const float*>(p.bias)[col + i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + i]);
          }
          if (p.out_f32) {
            float* c = reinterpret_cast<float*>(p.C) + off;
            if (whole && (reinterpret_cast<uintptr_t>(c) & 15) == 0) {
              float4 o = make_float4(v[0], v[1], v[2], v[3]);
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(c);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(c) = o;
            } else {
              for (int i = 0; i < 4 && col + i < p.N; ++i) c[i] = p.accumulate ? c[i] + v[i] : v[i];
            }
          } else {
            __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C) + off;
            if (whole && (reinterpret_cast<uintptr_t>(c) & 7) == 0) {
              if (p.accumulate) {
                const uint2 old = *reinterpret_cast<const uint2*>(c);
                const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&old.x));
                const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&old.y));
                v[0] += f0.x; v[1] += f0.y; v[2] += f1.x; v[3] += f1.y;
              }
              uint2 o;
              *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v[0], v[1]);
              *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v[2], v[3]);
              *reinterpret_cast<uint2*>(c) = o;
            } else {
              for (int i = 0; i < 4 && col + i < p.N; ++i)
                c[i] = __float2bfloat16(p.accumulate ? __bfloat162float(c[i]) + v[i] : v[i]);
            }
          }
        };
        for (int u = q; u < units; u += 8) {
          const int u2 = u + 4;
          const bool has2 = u2 < units;
          const int r1 = (u % row_blocks) * 32 + lane, r2 = (u2 % row_blocks) * 32 + lane;
          const bool ok1 = r1 < valid_rows, ok2 = has2 && r2 < valid_rows;
          const float* s1 = tile_ws + (size_t)(g0 + u / row_blocks) * (kBlockM * 4) + (size_t)r1 * 4;
          const float* s2 = tile_ws + (size_t)(g0 + (has2 ? u2 : u) / row_blocks) * (kBlockM * 4) + (size_t)r2 * 4;
          float4 a1 = zero4, a2 = zero4;
          for (int h0 = 0; h0 < w.nsplit; h0 += 8) {
            float4 t1[8], t2[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const bool in = h0 + j < w.nsplit;
              t1[j] = (in && ok1) ? __ldcg(reinterpret_cast<const float4*>(s1 + (size_t)(h0 + j) * part_stride)) : zero4;
              t2[j] = (in && ok2) ? __ldcg(reinterpret_cast<const float4*>(s2 + (size_t)(h0 + j) * part_stride)) : zero4;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              a1.x += t1[j].x; a1.y += t1[j].y; a1.z += t1[j].z; a1.w += t1[j].w;
              a2.x += t2[j].x; a2.y += t2[j].y; a2.z += t2[j].z; a2.w += t2[j].w;
            }
          }
          finish(u, a1);
          if (has2) finish(u2, a2);
        }
        __syncwarp();
        if (lane == 0) {
          // check-out: the last of the 4 * nsplit warps re-arms the flag (none can still be waiting)
          const unsigned old = atomicAdd(p.sk_flags + w.tail_idx, 1u);
          if (old == 8u * w.nsplit - 1u) p.sk_flags[w.tail_idx] = 0;
        }
        continue;
      }
      // split last wave with a fused reduce-scatter epilogue: helpers park their fp32 partial tile in the
      // workspace; the owner waits for them and folds them in below
      float* sk_tile = nullptr;
      if (w.nsplit > 1) {
        sk_tile = p.sk_ws + ((size_t)w.tail_idx * (w.nsplit - 1)) * (size_t)(kBlockM * BLOCK_N);
        if (w.split > 0) {
          // layout [column / 4][row][4]: the 32 lanes of a warp (32 rows) write 512 contiguous bytes
          float* dst = sk_tile + (size_t)(w.split - 1) * (kBlockM * BLOCK_N) + (size_t)(q * 32 + lane) * 4;
#pragma unroll 1
          for (int c = 0; c < BLOCK_N; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(dst + (size_t)((c + i) >> 2) * (kBlockM * 4)) =
                  make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                              __uint_as_float(r[i + 3]));
          }
          tc_fence_before_sync();
          __threadfence();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive(&tempty[as]);
            red_release_gpu_add(p.sk_flags + w.tail_idx, 1u);
          }
          continue;
        }
        // owner: all helpers (4 warps each) must have stored their partials
        bool got = true;
        if (lane == 0)
          got = flag_wait_ge(p.sk_flags + w.tail_idx, 4u * (w.nsplit - 1), false, p.status, p.wait_ns, 14);
        got = __all_sync(0xffffffffu, got);
        if (!got) { *abort_w = 1; break; }
      }
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
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (sk_tile) {
            for (int h = 0; h < w.nsplit - 1; ++h) {
              const float* src = sk_tile + (size_t)h * (kBlockM * BLOCK_N) + (size_t)(q * 32 + lane) * 4;
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 t4 = __ldcg(reinterpret_cast<const float4*>(src + (size_t)((c + i) >> 2) * (kBlockM * 4)));
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
                float b = p.bias_f32
                              ? reinterpret_cast<const float*>(p.bias)[col0 + i]
                              : __bfloat162float(
                                    reinterpret_cast<const __nv_bfloat16*>(p.bias)[col0 + i]);
                v[i] += b;
              }
            }
          }
          if (p.rs_mode && rs_coalesce) {
            // bf16 partial into the warp's staging rows; flushed below in 128-byte row segments
            uint8_t* srow = out_stage + lane * 144 + (c & 32) * 2;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j)
                ob2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
              *reinterpret_cast<uint4*>(srow + i * 2) = o;
            }
          } else if (p.rs_mode) {
            // row block -> owning rank; bf16 partial straight into that rank's staging slice
            const int d = row / p.rs_rows_per_rank;
            __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.rs_stage[d]) +
                                  ((size_t)p.rank * p.rs_rows_per_rank + (row - d * p.rs_rows_per_rank)) * p.N + col0;
            if (full_chunk) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint4 o;
                __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  ob2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(crow + i) = o;
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (col0 + i < p.N) crow[i] = __float2bfloat16(v[i]);
            }
          } else if (p.out_f32) {
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
        if (p.rs_mode && rs_coalesce && (c & 32)) {
          // two 32-column chunks are staged: each store instruction now writes 4 rows x 128
          // contiguous bytes (peer stores of whole cache lines instead of 16-byte fragments)
          __syncwarp();
          const int col64 = tn * BLOCK_N + (c - 32);
#pragma unroll
          for (int it4 = 0; it4 < 8; ++it4) {
            const int rr = it4 * 4 + (lane >> 3);
            const int grow = tm * kBlockM + q * 32 + rr;
            if (grow < p.M) {
              const uint4 val = *reinterpret_cast<const uint4*>(out_stage + rr * 144 + (lane & 7) * 16);
              const int d = grow / p.rs_rows_per_rank;
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.rs_stage[d]) +
                                   ((size_t)p.rank * p.rs_rows_per_rank + (grow - d * p.rs_rows_per_rank)) * p.N +
                                   col64 + (lane & 7) * 8;
              *reinterpret_cast<uint4*>(dst) = val;
            }
          }
          __syncwarp();
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[as]);
      if (sk_tile && lane == 0) {
        // each owner warp checks out after consuming the partials; the last one re-arms the flag
        // (no warp can still be waiting: checking out happens after passing the wait)
        const unsigned old = atomicAdd(p.sk_flags + w.tail_idx, 1u);
        if (old == 4u * (w.nsplit - 1) + 3u) p.sk_flags[w.tail_idx] = 0;
      }
      if (p.rs_mode) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          // one arrival per destination rank whose rows this warp's 32-row block touched
          const int r0 = tm * kBlockM + q * 32;
          const int r1 = min(r0 + 32, p.M) - 1;
          if (r1 >= r0)
            for (int d = r0 / p.rs_rows_per_rank; d <= r1 / p.rs_rows_per_rank; ++d)
              red_release_sys_add(p.rs_cnt[d] + p.rank, 1u);
        }
      }
    }
    if (p.rs_mode) rs_reduce_role(p, bid, nctas, (warp & 3) * 32 + lane, wc);
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

// 2-D int8 tensor map with 128-byte swizzle: inner dim `d0` contiguous (bytes), box = {128, box1}.
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t ld,
                    uint32_t box1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {d0, d1};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

#ifdef TPB_KERNEL_DEBUG
static DbgSetter g_dbg_setters[64];
static int g_dbg_n = 0;
void dbg_register_setter(DbgSetter fn) {
  if (g_dbg_n < 64) g_dbg_setters[g_dbg_n++] = fn;
}
#endif

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

// Split-K workspace (fp32 partial tiles + one flag per tail tile), registered by the caller once
// per device; GEMMs that use it must be stream-ordered with respect to each other.
static float* g_sk_ws = nullptr;
static uint32_t* g_sk_flags = nullptr;
void splitk_workspace(float** ws, uint32_t** flags) {
  *ws = g_sk_ws;
  *flags = g_sk_flags;
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
  // few tiles and a deep reduction: launch every SM and let the tail split along K
  if (p.sk_ws && tiles < max_ctas && tail_nsplit(tiles, max_ctas, (p.K + kBlockK - 1) / kBlockK) > 1) grid = max_ctas;
  grid += p.n_copy;
  if (grid <= 0) return 0;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

// Tile width: 256 columns, except when that leaves more than half of the SMs without a tile
// (small-M decode shapes): then 128-column tiles double the number of CTAs that stream weights.
// With the split-K workspace registered both widths are costed after their tiles are split along K
// (same rule as the kernel's schedule): what bounds a few-row product is the rate at which one SM
// fills its shared memory (about 100 GB/s), so the cost is the kilobytes one CTA brings in - k-blocks
// per split x (A box + B box) - plus the price of a split, in the same unit.
static int pick_block_n(int M, int N, int K, bool splitk) {
  if (N <= 128) return 128;
  const long long tm = (M + kBlockM - 1) / kBlockM;
  const long long tiles256 = tm * ((N + 255) / 256);
  if (tiles256 * 2 > sm_count()) return 256;
  if (!splitk) return 128;
  const int kb = (K + kBlockK - 1) / kBlockK;
  const int a_kb = M <= 64 ? 8 : 16;
  auto cost = [&](long long tiles, int b_kb) {
    const int ns = tiles < sm_count() ? tail_nsplit((int)tiles, sm_count(), kb) : 1;
    return (long long)((kb + ns - 1) / ns) * (a_kb + b_kb) + (ns > 1 ? 640 : 0);
  };
  return cost(tiles256, 32) <= cost(tm * ((N + 127) / 128), 16) ? 256 : 128;
}

int gemm_bf16_dispatch(const void* A, const void* B, void* C, const void* bias, int M, int N,
                       int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                       int bias_f32, int accumulate, float alpha, const uint32_t* b_flags,
                       int rows_per_flag, uint32_t flag_want, int max_ctas, uint32_t* status,
                       cudaStream_t stream, const GemmFused* fused) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  const int block_n = pick_block_n(M, N, K, g_sk_ws != nullptr && fused == nullptr);
  CUtensorMap ta, tb;
  int r;
  const int a_box_rows = (!a_mn && M <= 64) ? 64 : kBlockM;
  if (!a_mn) r = make_tmap_2d_bf16(&ta, A, K, M, lda, a_box_rows);
  else r = make_tmap_2d_bf16(&ta, A, M, K, lda, kBlockK);
  if (r) return r;
  if (!b_mn) r = make_tmap_2d_bf16(&tb, B, K, N, ldb, block_n);
  else r = make_tmap_2d_bf16(&tb, B, N, K, ldb, kBlockK);
  if (r) return r;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.a_box_rows = a_box_rows; p.ldc = ldc; p.C = C; p.bias = bias; p.bias_f32 = bias_f32;
  p.out_f32 = out_f32; p.accumulate = accumulate; p.alpha = alpha; p.status = status;
  p.wait_ns = kDefaultWaitNs;
  p.b_flags = b_flags; p.rows_per_flag = rows_per_flag > 0 ? rows_per_flag : 1;
  p.flag_want = flag_want;
  p.epoch_dev = nullptr; p.rs_per_call = 0;
  p.n_copy = 0; p.ag_operand = 0; p.rs_mode = 0; p.tile_m_shift = 0; p.tile_n_shift = 0; p.world = 1; p.rank = 0;
  p.sk_ws = g_sk_ws; p.sk_flags = g_sk_flags;
  if (fused) {
    p.n_copy = fused->n_copy; p.ag_operand = fused->ag_operand; p.world = fused->world;
    p.rank = fused->rank; p.ag_dst = fused->ag_dst; p.ag_shard_bytes = fused->ag_shard_bytes;
    p.ag_chunk_bytes = fused->ag_chunk_bytes; p.ag_rows_per_rank = fused->ag_rows_per_rank;
    p.ag_rows_per_flag = fused->ag_rows_per_flag; p.ag_flags = fused->ag_flags;
    p.pad_local = fused->pad_local; p.ready_slot = fused->ready_slot; p.done_slot = fused->done_slot;
    p.epoch = fused->epoch; p.epoch_dev = fused->epoch_dev; p.rs_per_call = fused->rs_per_call; p.tile_m_shift = fused->tile_m_shift; p.tile_n_shift = fused->tile_n_shift; p.rs_mode = fused->rs_mode;
    p.rs_rows_per_rank = fused->rs_rows_per_rank; p.rs_expect = fused->rs_expect;
    p.rs_out = fused->rs_out;
    for (int r = 0; r < 16; ++r) {
      p.ag_src[r] = fused->ag_src[r]; p.pad_peer[r] = fused->pad_peer[r];
      p.rs_stage[r] = fused->rs_stage[r]; p.rs_cnt[r] = fused->rs_cnt[r];
    }
    if (fused->wait_ns) p.wait_ns = fused->wait_ns;
  }
  if (max_ctas <= 0) max_ctas = sm_count();
  max_ctas -= p.n_copy;
  if (max_ctas < 1) return -2;
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

// Shapes that go to the CTA-pair kernel when nothing pins the choice: at least `g_pair_min_tiles`
// tiles of 256 x 256 (one full wave of CTA pairs by default), every operand layout. With both
// operands MN-major (weight gradients) the two kernels time the same in isolation, but the pair
// kernel moves a third less through shared memory and the training step, which runs at the power
// cap, is 1.2 % shorter with it. 0 = never.
static int g_pair_min_tiles = 74;
extern "C" void tpb_gemm_set_pair_min_tiles(int tiles) { g_pair_min_tiles = tiles; }

namespace tpb { int g_nvtx_on = 0; }
extern "C" void tpb_nvtx_enable(int on) { tpb::g_nvtx_on = on; }
extern "C" int tpb_nvtx_enabled() { return tpb::g_nvtx_on; }

// 1 if this library was built with index checks (TPB_KERNEL_DEBUG), and the word they report to.
extern "C" int tpb_debug_build() {
#ifdef TPB_KERNEL_DEBUG
  return 1;
#else
  return 0;
#endif
}
extern "C" int tpb_debug_set_status(uint32_t* status) {
#ifdef TPB_KERNEL_DEBUG
  for (int i = 0; i < tpb::g_dbg_n; ++i) {
    const int r = tpb::g_dbg_setters[i](status);
    if (r) return r;
  }
  return 0;
#else
  (void)status;
  return -1;
#endif
}

extern "C" int tpb_gemm_bf16_single(const void* A, const void* B, void* C, const void* bias, int M, int N,
                                    int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                                    int bias_f32, int accumulate, float alpha, uint32_t* status,
                                    void* stream) {
  TPB_NVTX("tpb_gemm_bf16_single");
  return tpb::gemm_bf16_dispatch(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32,
                                 bias_f32, accumulate, alpha, nullptr, 0, 0, 0, status,
                                 static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int tpb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N,
                             int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                             int bias_f32, int accumulate, float alpha, uint32_t* status,
                             void* stream) {
  TPB_NVTX("tpb_gemm_bf16");
  if (g_pair_min_tiles > 0 && (long long)((M + 255) / 256) * ((N + 255) / 256) >= g_pair_min_tiles)
    return tpb::gemm_pair_dispatch(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, bias_f32,
                                   accumulate, alpha, 0, status, static_cast<cudaStream_t>(stream));
  return tpb::gemm_bf16_dispatch(A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32,
                                 bias_f32, accumulate, alpha, nullptr, 0, 0, 0, status,
                                 static_cast<cudaStream_t>(stream), nullptr);
}

// ------------------------------------------------------------------ fused collectives (host)
// C[M, N] = gather_rows(A)[M, K] * B[N, K]^T where A is row-sharded over the ranks: rank r's
// rows [r * M/world, (r+1) * M/world) live in rank r's copy of the symmetric buffer at arena
// offset a_off (shape [M, K], ld = K); after the call the local copy holds all rows.
//   flags: local device array of at least world * ceil(shard_rows / rows_per_flag) + 1 words.
//   ready_slot / done_slot: `world` signal slots each; epoch must grow by one per call.
extern "C" int tpb_ag_gemm(size_t a_off, const void* B, void* C, const void* bias, int M, int N,
                           int K, int ldb, int ldc, int b_mn, int out_f32, uint32_t* flags,
                           int rows_per_flag, size_t pad_off, int ready_slot, int done_slot,
                           uint32_t epoch, int n_copy, double wait_s, uint32_t* status,
                           void* stream, const uint32_t* epoch_dev) {
  TPB_NVTX("tpb_ag_gemm");
  const tpb::SymmView* sv = tpb::symm_view();
  if (!sv || sv->world < 1 || M % sv->world) return -2;
  const int world = sv->world, rank = sv->rank;
  const int rows_per_rank = M / world;
  if (rows_per_rank % rows_per_flag) return -2;
  tpb::GemmFused f;
  memset(&f, 0, sizeof(f));
  f.world = world; f.rank = rank;
  f.n_copy = world > 1 ? (n_copy > 0 ? n_copy : 16) : 0;
  f.ag_operand = world > 1 ? 1 : 0;
  f.ag_shard_bytes = (unsigned long long)rows_per_rank * K * 2;
  f.ag_chunk_bytes = (unsigned long long)rows_per_flag * K * 2;
  f.ag_rows_per_rank = rows_per_rank; f.ag_rows_per_flag = rows_per_flag;
  f.ag_flags = flags;
  f.ag_dst = sv->peer[rank] + a_off;
  for (int r = 0; r < world; ++r) {
    f.ag_src[r] = sv->peer[r] + a_off + (size_t)r * f.ag_shard_bytes;
    f.pad_peer[r] = reinterpret_cast<uint32_t*>(sv->peer[r] + pad_off);
  }
  f.pad_local = reinterpret_cast<uint32_t*>(sv->peer[rank] + pad_off);
  f.ready_slot = ready_slot; f.done_slot = done_slot; f.epoch = epoch; f.epoch_dev = epoch_dev;
  const int tiles_m = (M + 127) / 128;
  f.tile_m_shift = (rows_per_rank % 128 == 0) ? (int)(((long long)rank * rows_per_rank / 128) % tiles_m) : 0;
  f.wait_ns = wait_s > 0 ? (unsigned long long)(wait_s * 1e9) : 0;
  return tpb::gemm_bf16_dispatch(sv->peer[rank] + a_off, B, C, bias, M, N, K, K, ldb, ldc, 0, b_mn,
                                 out_f32, 0, 0, 1.f, nullptr, 0, 0, 0, status,
                                 static_cast<cudaStream_t>(stream), &f);
}

// C[M, N] = A[M, K] * gather_rows(W)[N, K]^T where the WEIGHT is row-sharded over the ranks (a fully
// sharded parameter): rank r's rows [r * N/world, (r+1) * N/world) live in rank r's copy of the symmetric
// buffer at arena offset w_off (shape [N, K], ld = K); after the call the local copy holds all rows.
// Copy CTAs of the same launch pull the peers' shards while the tensor-core CTAs start on the tiles of
// the local rows; a tile of remote rows waits (bounded) for the flags of its row blocks.
// flags / slots / epoch as in tpb_ag_gemm.
extern "C" int tpb_ag_gemm_weight(const void* A, size_t w_off, void* C, const void* bias, int M, int N, int K,
                                  int lda, int ldc, int a_mn, int out_f32, uint32_t* flags, int rows_per_flag,
                                  size_t pad_off, int ready_slot, int done_slot, uint32_t epoch, int n_copy,
                                  double wait_s, uint32_t* status, void* stream, const uint32_t* epoch_dev) {
  TPB_NVTX("tpb_ag_gemm_weight");
  const tpb::SymmView* sv = tpb::symm_view();
  if (!sv || sv->world < 1 || N % sv->world) return -2;
  const int world = sv->world, rank = sv->rank;
  const int rows_per_rank = N / world;
  if (rows_per_flag <= 0 || rows_per_rank % rows_per_flag) return -2;
  tpb::GemmFused f;
  memset(&f, 0, sizeof(f));
  f.world = world; f.rank = rank;
  f.n_copy = world > 1 ? (n_copy > 0 ? n_copy : 16) : 0;
  f.ag_operand = world > 1 ? 2 : 0;
  f.ag_shard_bytes = (unsigned long long)rows_per_rank * K * 2;
  f.ag_chunk_bytes = (unsigned long long)rows_per_flag * K * 2;
  f.ag_rows_per_rank = rows_per_rank; f.ag_rows_per_flag = rows_per_flag;
  f.ag_flags = flags;
  f.ag_dst = sv->peer[rank] + w_off;
  for (int r = 0; r < world; ++r) {
    f.ag_src[r] = sv->peer[r] + w_off + (size_t)r * f.ag_shard_bytes;
    f.pad_peer[r] = reinterpret_cast<uint32_t*>(sv->peer[r] + pad_off);
  }
  f.pad_local = reinterpret_cast<uint32_t*>(sv->peer[rank] + pad_off);
  f.ready_slot = ready_slot; f.done_slot = done_slot; f.epoch = epoch; f.epoch_dev = epoch_dev;
  const int block_n = tpb::pick_block_n(M, N, K, false);
  const int tiles_n = (N + block_n - 1) / block_n;
  f.tile_n_shift = (rows_per_rank % block_n == 0) ? (int)(((long long)rank * rows_per_rank / block_n) % tiles_n) : 0;
  f.wait_ns = wait_s > 0 ? (unsigned long long)(wait_s * 1e9) : 0;
  return tpb::gemm_bf16_dispatch(A, sv->peer[rank] + w_off, C, bias, M, N, K, lda, K, ldc, a_mn, 0, out_f32, 0, 0,
                                 1.f, nullptr, 0, 0, 0, status, static_cast<cudaStream_t>(stream), &f);
}

// out[M/world, N] (local) = sum over ranks of (A_r[M, K] * B_r[N, K]^T)[rows of this rank].
// stage_off: arena offset of a [world, M/world, N] bf16 staging buffer; cnt_slot: `world`
// signal slots used as tile counters (monotonic; `expect` = value meaning "all arrived").
extern "C" int tpb_gemm_rs(const void* A, const void* B, void* out, int M, int N, int K, int lda,
                           int ldb, int a_mn, int b_mn, size_t stage_off, size_t pad_off,
                           int cnt_slot, uint32_t epoch, double wait_s, uint32_t* status,
                           void* stream, const uint32_t* epoch_dev) {
  TPB_NVTX("tpb_gemm_rs");
  const tpb::SymmView* sv = tpb::symm_view();
  if (!sv || sv->world < 1 || M % sv->world || N % 8) return -2;
  const int world = sv->world, rank = sv->rank;
  tpb::GemmFused f;
  memset(&f, 0, sizeof(f));
  f.world = world; f.rank = rank;
  f.rs_mode = 1;
  f.rs_rows_per_rank = M / world;
  for (int r = 0; r < world; ++r) {
    f.rs_stage[r] = sv->peer[r] + stage_off;
    f.rs_cnt[r] = reinterpret_cast<uint32_t*>(sv->peer[r] + pad_off) + cnt_slot;
  }
  const int block_n = tpb::pick_block_n(M, N, K, false);
  // arrivals this rank expects from each source per call: one per (N tile, 32-row block that
  // overlaps this rank's rows)
  const int my0 = rank * f.rs_rows_per_rank, my1 = my0 + f.rs_rows_per_rank - 1;
  const int row_blocks = my1 / 32 - my0 / 32 + 1;
  const int per_call = row_blocks * ((N + block_n - 1) / block_n);
  f.rs_expect = epoch * (uint32_t)per_call;
  f.epoch = epoch; f.epoch_dev = epoch_dev; f.rs_per_call = (uint32_t)per_call;
  f.rs_out = static_cast<__nv_bfloat16*>(out);
  const int tiles_m = (M + 127) / 128;
  f.tile_m_shift = (f.rs_rows_per_rank % 128 == 0)
                       ? (int)(((long long)((rank + 1) % world) * f.rs_rows_per_rank / 128) % tiles_m)
                       : 0;
  f.wait_ns = wait_s > 0 ? (unsigned long long)(wait_s * 1e9) : 0;
  return tpb::gemm_bf16_dispatch(A, B, nullptr, nullptr, M, N, K, lda, ldb, N, a_mn, b_mn, 0, 0, 0,
                                 1.f, nullptr, 0, 0, 0, status, static_cast<cudaStream_t>(stream),
                                 &f);
}

// Bytes of fp32 workspace and number of flag words that tpb_gemm_set_splitk_workspace expects.
extern "C" long long tpb_gemm_splitk_workspace_bytes() {
  return (long long)tpb::sm_count() * 128 * 256 * 4;
}
// ws: tpb_gemm_splitk_workspace_bytes() bytes; flags: sm_count() zero-initialised uint32 words.
// Passing null disables the split of the last wave.
extern "C" int tpb_gemm_set_splitk_workspace(void* ws, uint32_t* flags) {
  tpb::g_sk_ws = static_cast<float*>(ws);
  tpb::g_sk_flags = flags;
  return 0;
}
