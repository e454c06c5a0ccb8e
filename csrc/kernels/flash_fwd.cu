// Flash attention forward for sm_100a: GQA-native, causal or full, head_dim 64 / 128.
//
// One CTA handles two tiles of 128 queries of one query head in ping-pong. Warp 0 streams K/V
// tiles with TMA through one ring, warp 1 issues tcgen05.mma: S_g = Q_g K^T into the TMEM region
// of tile g and O_g += P_g V into a second region; each tile has four softmax warps with one
// query row per thread: they read S from TMEM, keep the running max / sum in the exp2 domain,
// write P (bf16 pairs) back over the S columns - the second MMA takes P as its A operand
// straight from TMEM - rescale O in TMEM only when a row maximum grew by more than a factor of two, and
// finally write O / LSE. While one tile is in its softmax the tensor pipe runs the other tile's
// MMAs. K and V of a KV head are shared by the query heads of its group through L2, so GQA costs
// no expanded K/V traffic.
//
// Counterpart in the reference: vendored FlashAttention-2 sm80 leaves
// (p10/src/backend/cuda/transformers/flash/flash_fwd_kernel.h, AttentionKernels.cu:1782-1969),
// which expand K/V to the query head count for GQA training (nn/functional.py:3571-3586).
#include "sm100.cuh"
#include "tpb_api.h"

#include <mutex>

namespace tpb {

constexpr int kAttnThreads = 320;  // TMA warp, MMA warp, 2 x 4 softmax warps (one group per query tile)
constexpr int kBlockQ = 128;
constexpr int kTilesQ = 2;  // query tiles per CTA, processed in ping-pong
constexpr int kBlockKV = 128;
constexpr float kNegBig = -1.0e30f;

struct AttnFwdParams {
  int B, Tq, Tk, Hq, Hkv;
  int causal;
  int kv_offset;  // causal: query i attends keys <= i + kv_offset (Tk - Tq)
  float scale_log2e;
  __nv_bfloat16* O;
  long long o_tok_stride, o_head_stride, o_batch_stride;
  float* lse;  // [B, Hq, lse_stride]
  int lse_stride;
  const int* kv_len;  // optional device word: number of valid keys (<= Tk), for graph-replayed decode
  // Optional lower / upper bounds of the keys of a query (local attention and packed sequences):
  //   window > 0: query i attends keys > i + kv_offset - window;
  //   seg_start / seg_end [B * Tq] (null = none): query i attends keys in [seg_start[i], seg_end[i]);
  //   both arrays are non-decreasing along a sequence (segments are contiguous token ranges).
  int window;
  const int* seg_start;
  const int* seg_end;
  // split-KV (decode): CTA (x = tile * n_splits + split) handles KV blocks [split * blocks_per_split, ...)
  // and writes a partial O / LSE at split * o_split_stride / lse_split_stride (merged by a second kernel)
  int n_splits, blocks_per_split;
  long long o_split_stride, lse_split_stride;
  uint32_t* status;
  unsigned long long wait_ns;
  unsigned long long* trace;  // optional: cycle stamps of CTA (0,0,0), see tpb_flash_fwd_set_trace
  int trace_cap;
};

// Debug aid: cycle stamps of block (0,0,0), kept in shared memory while the kernel runs (a stamp
// costs one shared store) and copied out at the end: trace[(who * 64 + it) * 8 + tag] = clock.
//   who 0: MMA thread (tags 0/1: P half of tile 0/1 seen, 2/3: P complete, 4/5: S(j+1) issued)
//   who 1/2: first softmax thread of tile 0/1 (tags 1: S seen, 2: S in registers, 3: maximum done,
//            4: first half exponentiated, 5: first half handed over, 6: second half exponentiated,
//            7: second half handed over)
constexpr int kTraceIts = 64;
constexpr int kTraceWords = 3 * kTraceIts * 8;
__device__ __forceinline__ void fwd_trace(uint32_t* tr, int who, int tag, int it) {
  if (tr && it < kTraceIts) tr[(who * kTraceIts + it) * 8 + tag] = (uint32_t)clock64();
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // pure: let the compiler schedule it
  return y;
}

// Packed fp32x2 arithmetic on 64-bit register pairs (one issue slot for two elements).
__device__ __forceinline__ uint64_t pk2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ uint64_t pk2u(uint32_t a, uint32_t b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2_down(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// Maximum of one S row (raw scores): four chains of three-input maxima.
__device__ __forceinline__ float row_max(const uint32_t (&sr)[128]) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int i = 0; i < 128; i += 8) {
    m0 = max3(m0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
    m1 = max3(m1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
    m2 = max3(m2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
    m3 = max3(m3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// Keys outside [lo, lim] get the score -inf (masked tiles only: the diagonal, the ragged end of the
// sequence, the left edge of a window or segment): it never raises the running maximum and its
// exponential on the special-function unit is exactly zero, also for a row without any valid key
// in this tile.
__device__ __forceinline__ void row_mask(uint32_t (&sr)[128], int k0, int lo, int lim) {
  const int a = lo - k0, b = lim - k0;   // valid columns: a <= i <= b
#pragma unroll
  for (int i = 0; i < 128; ++i) sr[i] = (i >= a && i <= b) ? sr[i] : 0xff800000u;
}

// exp2 of a pair on the FMA pipe: floor by the magic-number add in round-down mode, cubic
// polynomial on the fraction (relative error 1e-4, below the bf16 rounding of P), exponent added
// as an integer. The special-function unit delivers 16 exp2 per cycle and SM while the tensor pipe
// needs 16 per cycle for 128-wide head dimensions, so a share of the row goes this way.
__device__ __forceinline__ uint64_t exp2_poly2(uint64_t x) {
  float x0, x1;
  upk2(x, x0, x1);
  const uint64_t xc = pk2(fmaxf(x0, -127.f), fmaxf(x1, -127.f));
  const uint64_t magic = pk2(12582912.f, 12582912.f);  // 2^23 + 2^22
  const uint64_t r = add2_down(xc, magic);
  const uint64_t fr = sub2(xc, sub2(r, magic));
  uint64_t pl = fma2(fr, pk2(0.077119089663028717f, 0.077119089663028717f), pk2(0.227564394474029541f, 0.227564394474029541f));
  pl = fma2(pl, fr, pk2(0.695146143436431885f, 0.695146143436431885f));
  pl = fma2(pl, fr, pk2(1.f, 1.f));
  uint32_t p0, p1, r0, r1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(p0), "=r"(p1) : "l"(pl));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(r0), "=r"(r1) : "l"(r));
  return pk2u(p0 + (r0 << 23), p1 + (r1 << 23));
}

// One half of a row: columns [HALF * 64, HALF * 64 + 64) of sr become 32 bf16 pairs
// P = exp2(S * scale - m) in sr[HALF * 32 ...] (in place: the pairs land where scores were already
// consumed); the fp32 values are added into two packed accumulators. Of every four column pairs,
// NPOLY take the polynomial, the rest the special-function unit.
template <int HALF, int NPOLY>
__device__ __forceinline__ void row_exp_half(uint32_t (&sr)[128], uint64_t sc, uint64_t nm, uint64_t& acc0,
                                             uint64_t& acc1) {
#pragma unroll
  for (int i = HALF * 32; i < HALF * 32 + 32; ++i) {
    const uint64_t x = fma2(pk2u(sr[2 * i], sr[2 * i + 1]), sc, nm);
    uint64_t e;
    if ((i & 3) < NPOLY) {
      e = exp2_poly2(x);
    } else {
      float x0, x1;
      upk2(x, x0, x1);
      e = pk2(fast_exp2(x0), fast_exp2(x1));
    }
    if (i & 1) acc1 = add2(acc1, e);
    else acc0 = add2(acc0, e);
    float e0, e1;
    upk2(e, e0, e1);
    sr[i] = pack_bf16(e0, e1);
  }
}

template <int D>
struct AttnSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kQBytes = kBlockQ * D * 2;   // one Q tile
  static constexpr int kKBytes = kBlockKV * D * 2;  // one K or V tile
  static constexpr int kQOff = 0;                   // two Q tiles
  // K and V tiles share one ring (K0 V0 K1 V1 ...)
  static constexpr int kRing = D == 128 ? 4 : 6;
  static constexpr int kKOff = kQOff + kTilesQ * kQBytes;
  static constexpr int kBarOff = kKOff + kRing * kKBytes;
  static constexpr int kTraceOff = kBarOff + 256;
  static constexpr int kTotal = kTraceOff + kTraceWords * 4 + 1024;
  static_assert(kTotal <= 227 * 1024, "attention forward exceeds the shared memory of one CTA");
};

template <int D, int NPOLY>
__global__ void __launch_bounds__(kAttnThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using L = AttnSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  constexpr int R = L::kRing;
  uint64_t* q_full = bars;              // 1
  uint64_t* kv_full = bars + 1;         // R
  uint64_t* kv_empty = kv_full + R;     // R
  uint64_t* s_full = kv_empty + R;      // 2: S of tile g is complete (and so is every earlier MMA)
  uint64_t* p_half = s_full + 2;        // 2 (128 arrivals): keys 0..63 of P of tile g are in TMEM (and O is rescaled)
  uint64_t* p_full = p_half + 2;        // 2 (128 arrivals): all of P of tile g is in TMEM
  uint64_t* o_done = p_full + 2;        // 2: last PV of tile g is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 2);
  volatile uint32_t* abort_w = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_splits = p.n_splits > 1 ? p.n_splits : 1;
  const int q_tiles = gridDim.x / n_splits;
  int split, qt, h, b;
  if (p.causal && n_splits == 1) {
    // CTAs start in the order of their linear index. With a causal mask the work of a CTA grows with
    // its query tile, so the tile index is made the slowest coordinate, heaviest first, and the heads
    // of all batches the fastest: the light CTAs of every head come last and fill the tail evenly
    // (tile-major order within each head left the last head's CTAs to a few SMs).
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int hb = gridDim.y * gridDim.z;
    split = 0;
    qt = lin / hb;
    h = (lin % hb) % gridDim.y;
    b = (lin % hb) / gridDim.y;
  } else {
    split = blockIdx.x % n_splits;
    qt = blockIdx.x / n_splits;
    h = blockIdx.y;
    b = blockIdx.z;
  }
  const int qb = p.causal ? (q_tiles - 1 - qt) : qt;  // heavy tiles first
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qb * (kTilesQ * kBlockQ);
  const int Tk = p.kv_len ? min(p.Tk, *p.kv_len) : p.Tk;
  // first KV block of this CTA: the split's share, or the block of the smallest key that the CTA's
  // first query may attend (bounds grow with the query index, so later rows need no earlier key)
  int j0 = split * p.blocks_per_split;
  if (n_splits == 1 && q0 < p.Tq) {
    int lo_first = 0;
    if (p.window > 0) lo_first = max(lo_first, q0 + p.kv_offset - p.window + 1);
    if (p.seg_start) lo_first = max(lo_first, p.seg_start[(long long)b * p.Tq + q0]);
    j0 = lo_first / kBlockKV;
  }
  // KV blocks needed by each of the two query tiles
  int nkv_t[kTilesQ];
  int nkv = 0;
#pragma unroll
  for (int g = 0; g < kTilesQ; ++g) {
    int n = (Tk + kBlockKV - 1) / kBlockKV;
    if (p.causal) {
      const int last_key = q0 + g * kBlockQ + kBlockQ - 1 + p.kv_offset;
      n = last_key < 0 ? 0 : min(n, last_key / kBlockKV + 1);
    }
    if (q0 + g * kBlockQ >= p.Tq) n = 0;  // tile past the end of the sequence
    if (p.seg_end && n > 0) {
      // the tile's last query has the largest upper bound
      const int qlast = min(q0 + g * kBlockQ + kBlockQ - 1, p.Tq - 1);
      n = min(n, (p.seg_end[(long long)b * p.Tq + qlast] + kBlockKV - 1) / kBlockKV);
    }
    if (n_splits > 1) n = max(0, min(n - j0, p.blocks_per_split));  // this split's share
    else n = max(0, n - j0);
    nkv_t[g] = n;
    nkv = max(nkv, n);
  }

  if (threadIdx.x == 0) {
    *abort_w = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < R; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    for (int i = 0; i < kTilesQ; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_half[i], 128);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
    }
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
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
  uint32_t* trc = (p.trace && qt == 0 && h == 0 && b == 0)
                      ? reinterpret_cast<uint32_t*>(smem + L::kTraceOff) : nullptr;
  if (trc) {
    for (int i = threadIdx.x; i < kTraceWords; i += kAttnThreads) trc[i] = 0;
    __syncthreads();
    if (threadIdx.x == 0) fwd_trace(trc, 0, 1, 63);  // set-up done (slot 63 of the MMA row: CTA-level stamps)
  }

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && nkv > 0) {
      mbar_arrive_expect_tx(q_full, kTilesQ * L::kQBytes);
#pragma unroll
      for (int g = 0; g < kTilesQ; ++g)
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_4d(smem + L::kQOff + g * L::kQBytes + c * (kBlockQ * 128), &tmQ, q_full, c * 64, h,
                      q0 + g * kBlockQ, b);
      for (int t = 0; t < 2 * nkv; ++t) {
        const int j = t >> 1;
        const int slot = t % R;
        const uint32_t ph = (t / R) & 1;
        if (!mbar_wait_relaxed(&kv_empty[slot], ph ^ 1, wc, 1)) break;
        mbar_arrive_expect_tx(&kv_full[slot], L::kKBytes);
        const CUtensorMap* tm = (t & 1) ? &tmV : &tmK;
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c)
          tma_load_4d(smem + L::kKOff + slot * L::kKBytes + c * (kBlockKV * 128), tm, &kv_full[slot],
                      c * 64, hk, (j0 + j) * kBlockKV, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // Order on the tensor pipe: S0(0) S1(0) | PV0(0) S0(1) PV1(0) S1(1) | PV0(1) S0(2) ...
    // While the softmax warps of one tile work, the pipe runs the other tile's MMAs. P(j) lives
    // in the columns of S(j); S(j+1) is issued after PV(j) and the pipe executes in issue order,
    // so the overwrite needs no barrier.
    // The whole warp runs this loop with uniform control flow and one elected lane issues: operands of
    // tcgen05 instructions live in uniform registers, and inside a divergent `if (lane == 0)` region
    // every one of them would first be moved there from a vector register, which costs the issuing
    // thread about as many cycles as a 128 x 128 x 16 MMA takes to execute.
    if (nkv > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kBlockQ, kBlockKV, 1, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_f16(kBlockQ, D, 1, 0, 1);
      // descriptor words: the high words are constants, the low words are a base plus a constant per k-step
      constexpr uint32_t hi_k = smem_desc_hi(1024);  // K-major Q / K tiles and the MN-major V tile alike
      const uint32_t q_lo = smem_desc_lo(smem_u32(smem + L::kQOff), 16);
      const uint32_t k_lo = smem_desc_lo(smem_u32(smem + L::kKOff), 16);
      const uint32_t v_lo = smem_desc_lo(smem_u32(smem + L::kKOff), kBlockKV * 128);
      auto issue_s = [&](int g, int j) {
        const int slot = (2 * j) % R;
        const uint32_t qb_lo = q_lo + g * (L::kQBytes >> 4);
        const uint32_t kb_lo = k_lo + slot * (L::kKBytes >> 4);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = ((kk / 4) * (kBlockQ * 128) + (kk % 4) * 32) >> 4;
            umma_f16_ss_w(tmem_base + g * 128, qb_lo + off, hi_k, kb_lo + off, hi_k, idesc_s, kk != 0);
          }
          umma_commit(&s_full[g]);
        }
        __syncwarp();
      };
      auto commit = [&](uint64_t* bar) {
        if (elect_one()) umma_commit(bar);
        __syncwarp();
      };
      bool ok = mbar_wait_warp(q_full, 0, wc, 5);
      if (ok) ok = mbar_wait_warp(&kv_full[0], 0, wc, 3);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < kTilesQ; ++g)
          if (nkv_t[g] > 0) issue_s(g, 0);
        commit(&kv_empty[0]);
      }
      for (int j = 0; j < nkv && ok; ++j) {
        const int vslot = (2 * j + 1) % R;
        const uint32_t vph = ((2 * j + 1) / R) & 1;
        const int kslot = (2 * j + 2) % R;
        const uint32_t kph = ((2 * j + 2) / R) & 1;
        const uint32_t vb_lo = v_lo + vslot * (L::kKBytes >> 4);
        bool have_v = false, have_k = false;
#pragma unroll
        for (int g = 0; g < kTilesQ; ++g) {
          if (j >= nkv_t[g]) continue;
          // PV starts on the first 64 keys while the softmax warps still work on the other 64
          if (!mbar_wait_warp(&p_half[g], j & 1, wc, 6)) { ok = false; break; }
          if (lane == 0) fwd_trace(trc, 0, g, j);
          if (!have_v) {
            if (!mbar_wait_warp(&kv_full[vslot], vph, wc, 7)) { ok = false; break; }
            have_v = true;
          }
          tc_fence_after_sync();
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < kBlockKV / 32; ++kk)
              umma_f16_ts_w(tmem_base + 256 + g * 128, tmem_base + g * 128 + kk * 8, vb_lo + kk * (2048 >> 4), hi_k,
                            idesc_o, (j | kk) != 0);
          }
          __syncwarp();
          if (!mbar_wait_warp(&p_full[g], j & 1, wc, 11)) { ok = false; break; }
          if (lane == 0) fwd_trace(trc, 0, 2 + g, j);
          tc_fence_after_sync();
          if (elect_one()) {
#pragma unroll
            for (int kk = kBlockKV / 32; kk < kBlockKV / 16; ++kk)
              umma_f16_ts_w(tmem_base + 256 + g * 128, tmem_base + g * 128 + kk * 8, vb_lo + kk * (2048 >> 4), hi_k,
                            idesc_o, 1);
          }
          __syncwarp();
          if (j + 1 < nkv_t[g]) {
            if (!have_k) {
              if (!mbar_wait_warp(&kv_full[kslot], kph, wc, 3)) { ok = false; break; }
              have_k = true;
              tc_fence_after_sync();
            }
            if (g == 0 && lane == 0) fwd_trace(trc, 0, 6, j);
            issue_s(g, j + 1);
            if (g == 0 && lane == 0) fwd_trace(trc, 0, 7, j);
            if (lane == 0) fwd_trace(trc, 0, 4 + g, j);
          } else {
            commit(&o_done[g]);
          }
        }
        if (!ok) break;
        commit(&kv_empty[vslot]);
        if (have_k) commit(&kv_empty[kslot]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue
    // warps 2..5 own query tile 0, warps 6..9 tile 1; one query row per thread
    const int g = (warp - 2) >> 2;
    const int qd = warp & 3;
    const int row = qd * 32 + lane;  // row inside the tile == TMEM lane
    const int qi = q0 + g * kBlockQ + row;
    const uint32_t t_s = tmem_base + ((uint32_t)(qd * 32) << 16) + g * 128;
    const uint32_t t_o = tmem_base + ((uint32_t)(qd * 32) << 16) + 256 + g * 128;
    const int my_nkv = nkv_t[g];
    int lim = p.causal ? min(qi + p.kv_offset, Tk - 1) : (Tk - 1);  // last valid key
    int lo = 0;                                                            // first valid key
    // largest lower / smallest upper bound among the tile's rows decide which KV blocks need the mask
    int lo_tile = 0, lim_tile = 0x3fffffff;
    if (p.window > 0) {
      lo = qi + p.kv_offset - p.window + 1;
      lo_tile = q0 + g * kBlockQ + kBlockQ - 1 + p.kv_offset - p.window + 1;
    }
    if (p.seg_start) {
      const long long base = (long long)b * p.Tq;
      lo = max(lo, p.seg_start[base + min(qi, p.Tq - 1)]);
      lo_tile = max(lo_tile, p.seg_start[base + min(q0 + g * kBlockQ + kBlockQ - 1, p.Tq - 1)]);
    }
    if (p.seg_end) {
      const long long base = (long long)b * p.Tq;
      lim = min(lim, p.seg_end[base + min(qi, p.Tq - 1)] - 1);
      lim_tile = p.seg_end[base + min(q0 + g * kBlockQ, p.Tq - 1)] - 1;
    }
    float m = kNegBig, l = 0.f;
    bool ok = true;
    for (int j = 0; j < my_nkv; ++j) {
      if (!mbar_wait_warp(&s_full[g], j & 1, wc, 8)) { ok = false; break; }
      const bool tr = (threadIdx.x & 127) == 64;  // first thread of each tile's first softmax warp
      if (tr) fwd_trace(trc, 1 + g, 1, j);
      tc_fence_after_sync();
      const int k0 = (j0 + j) * kBlockKV;
      const bool need_mask = (p.causal && (k0 + kBlockKV - 1 > q0 + g * kBlockQ + p.kv_offset)) ||
                             (k0 + kBlockKV > Tk) || (k0 < lo_tile) || (k0 + kBlockKV - 1 > lim_tile);
      // the whole S row (128 fp32) in one TMEM round trip
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32(t_s + c * 32, &sr[c * 32]);
      tmem_ld_wait();
      if (tr) fwd_trace(trc, 1 + g, 2, j);
      if (need_mask) row_mask(sr, k0, lo, lim);
      const float mx = fmaxf(m, row_max(sr) * p.scale_log2e);
      // The reference maximum only moves when the row maximum grew by more than 2^4: until then
      // P stays below 16 (harmless in bf16, whose error is relative) and O needs no rescale.
      float alpha = 1.f;
      if (mx - m > 4.f) {
        alpha = fast_exp2(m - mx);
        m = mx;
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // every MMA issued before S(j), PV(j-1) included, completed before s_full fired
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(t_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32b_x16(t_o + c * 32, &o[0]);
          tmem_st_32x32b_x16(t_o + c * 32 + 16, &o[16]);
        }
      }
      // P = exp2(S * scale - m) as bf16 pairs written over the first 64 columns of S, in two halves
      // of 64 keys; the row sum adds the fp32 values
      const uint64_t sc2 = pk2(p.scale_log2e, p.scale_log2e), nm2 = pk2(-m, -m);
      uint64_t acc0 = pk2(0.f, 0.f), acc1 = acc0;
      if (tr) fwd_trace(trc, 1 + g, 3, j);
      // (masked tiles stay on the special-function unit, whose exp2(-inf) is an exact zero)
      if (need_mask) row_exp_half<0, 0>(sr, sc2, nm2, acc0, acc1);
      else row_exp_half<0, NPOLY>(sr, sc2, nm2, acc0, acc1);
      if (tr) fwd_trace(trc, 1 + g, 4, j);
      tmem_st_32x32b_x16(t_s, &sr[0]);
      tmem_st_32x32b_x16(t_s + 16, &sr[16]);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_half[g]);
      if (tr) fwd_trace(trc, 1 + g, 5, j);
      if (need_mask) row_exp_half<1, 0>(sr, sc2, nm2, acc0, acc1);
      else row_exp_half<1, NPOLY>(sr, sc2, nm2, acc0, acc1);
      if (tr) fwd_trace(trc, 1 + g, 6, j);
      tmem_st_32x32b_x16(t_s + 32, &sr[32]);
      tmem_st_32x32b_x16(t_s + 48, &sr[48]);
      float s0, s1;
      upk2(add2(acc0, acc1), s0, s1);
      l = l * alpha + (s0 + s1);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&p_full[g]);
      if (tr) fwd_trace(trc, 1 + g, 7, j);
    }
    if (ok && my_nkv > 0) ok = mbar_wait_warp(&o_done[g], 0, wc, 10);
    if ((threadIdx.x & 127) == 64) fwd_trace(trc, 0, 2 + g, 63);  // last PV of the tile complete
    if (ok) {
      tc_fence_after_sync();
      const float inv = (my_nkv > 0 && l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + split * p.o_split_stride + (long long)b * p.o_batch_stride + (long long)qi * p.o_tok_stride +
                            (long long)h * p.o_head_stride;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (my_nkv > 0) {
          tmem_ld_32x32b_x32(t_o + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (qi < p.Tq) {
#pragma unroll
          for (int gg = 0; gg < 4; ++gg) {
            uint4 v;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(o[gg * 8 + 0]) * inv,
                                                      __uint_as_float(o[gg * 8 + 1]) * inv);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(o[gg * 8 + 2]) * inv,
                                                      __uint_as_float(o[gg * 8 + 3]) * inv);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(o[gg * 8 + 4]) * inv,
                                                      __uint_as_float(o[gg * 8 + 5]) * inv);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(o[gg * 8 + 6]) * inv,
                                                      __uint_as_float(o[gg * 8 + 7]) * inv);
            v.x = *reinterpret_cast<uint32_t*>(&t0);
            v.y = *reinterpret_cast<uint32_t*>(&t1);
            v.z = *reinterpret_cast<uint32_t*>(&t2);
            v.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(orow + c * 32 + gg * 8) = v;
          }
        }
      }
      if (qi < p.Tq && p.lse) {
        float lse = (my_nkv > 0 && l > 0.f) ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        p.lse[split * p.lse_split_stride + ((long long)b * p.Hq + h) * p.lse_stride + qi] = lse;
      }
    }
  }

  if ((threadIdx.x & 127) == 64 && warp >= 2) fwd_trace(trc, 0, 4 + ((warp - 2) >> 2), 63);  // output written
  tc_fence_before_sync();
  __syncthreads();
  if (trc)
    for (int i = threadIdx.x; i < kTraceWords && i < p.trace_cap; i += kAttnThreads) p.trace[i] = trc[i];
  if (*abort_w) {
    unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// General bf16 tensor map: dims/strides innermost first (strides in elements; strides[0] must
// be 1 and is ignored), 128-byte swizzle or none.
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_elems, const uint32_t* box, int swizzle128) {
  ensure_thread_context();
  static EncodeTiledFn2 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn2>(sym);
  });
  if (!fn) return -1;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) st[i - 1] = strides_elems[i] * 2;
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), d, st, bx,
                  es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Tensor map over a [B, T, H, D] bf16 tensor given by strides; box = 64 (D) x 1 x rows x 1.
int make_tmap_bthd(CUtensorMap* out, const void* base, int B, int T, int H, int D,
                   long long tok_stride, long long head_stride, long long batch_stride, int rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)T, (uint64_t)B};
  uint64_t strides[4] = {1, (uint64_t)head_stride, (uint64_t)tok_stride, (uint64_t)batch_stride};
  uint32_t box[4] = {64, 1, (uint32_t)rows, 1};
  return make_tmap_bf16(out, base, 4, dims, strides, box, 1);
}

template <int D, int NPOLY>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const AttnFwdParams& p, cudaStream_t stream) {
  using L = AttnSmem<D>;
  auto kern = flash_fwd_kernel<D, NPOLY>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(((p.Tq + kTilesQ * kBlockQ - 1) / (kTilesQ * kBlockQ)) * (p.n_splits > 1 ? p.n_splits : 1), p.Hq, p.B);
  kern<<<grid, kAttnThreads, L::kTotal, stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

// Merge of split-KV partials: out[b, t, h, :] = sum_s w_s * part[s][b, t, h, :] with
// w_s = exp(lse_s - lse), lse = log sum_s exp(lse_s). One warp per (b, t, h).
__global__ void __launch_bounds__(256)
attn_split_merge_kernel(const __nv_bfloat16* __restrict__ part, const float* __restrict__ lse_part,
                        __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int n_splits, int B,
                        int T, int H, int D, long long part_split_stride, long long lse_split_stride,
                        int lse_stride, long long o_tok, long long o_head, long long o_batch) {
  const long long w = ((long long)blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * T * H) return;
  const int h = (int)(w % H);
  const long long bt = w / H;
  const int t = (int)(bt % T);
  const int b = (int)(bt / T);
  const long long li = ((long long)b * H + h) * lse_stride + t;
  float mx = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mx = fmaxf(mx, lse_part[s * lse_split_stride + li]);
  float den = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float l = lse_part[s * lse_split_stride + li];
    den += (l == -INFINITY) ? 0.f : __expf(l - mx);
  }
  const long long row = ((long long)(b * (long long)T + t) * H + h) * D;  // partials are contiguous [B, T, H, D]
  for (int d = lane * 2; d < D; d += 64) {
    float2 acc = make_float2(0.f, 0.f);
    for (int s = 0; s < n_splits; ++s) {
      const float l = lse_part[s * lse_split_stride + li];
      if (l == -INFINITY) continue;
      const float wgt = __expf(l - mx) / den;
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(part + s * part_split_stride + row + d));
      acc.x += wgt * v.x;
      acc.y += wgt * v.y;
    }
    *reinterpret_cast<__nv_bfloat162*>(out + b * o_batch + t * o_tok + h * o_head + d) = __floats2bfloat162_rn(acc.x, acc.y);
  }
  if (lane == 0 && lse_out) lse_out[li] = (den > 0.f) ? mx + __logf(den) : -INFINITY;
}

}  // namespace tpb

using namespace tpb;

static int g_fwd_npoly = 1;
static unsigned long long* g_fwd_trace = nullptr;
static int g_fwd_trace_cap = 0;

// Debug aid: buf = device array of `cap` uint64 (3 * 64 * 8 are used). The next forward launches
// copy the cycle stamps of block (0,0,0) into it (layout at fwd_trace). Pass null to switch it off.
extern "C" int tpb_flash_fwd_set_trace(unsigned long long* buf, int cap) {
  g_fwd_trace = buf;
  g_fwd_trace_cap = cap;
  return 0;
}

// q: [B, Tq, Hq, D], k/v: [B, Tk, Hkv, D] given by (token, head, batch) strides in elements;
// o likewise; lse: [B, Hq, lse_stride] fp32 (lse_stride >= Tq). causal aligns the last query with the last key.
// window > 0: local attention (a query attends its last `window` keys); seg_start / seg_end: int32
// [B * Tq] bounds [start, end) of the keys of every query (packed sequences; null = none).
extern "C" int tpb_flash_fwd_ex(const void* q, const void* k, const void* v, void* o, float* lse,
                                int B, int Tq, int Tk, int Hq, int Hkv, int D, long long q_tok,
                                long long q_head, long long q_batch, long long k_tok,
                                long long k_head, long long k_batch, long long v_tok,
                                long long v_head, long long v_batch, long long o_tok,
                                long long o_head, long long o_batch, int lse_stride, int causal,
                                float scale, uint32_t* status, void* stream, const int* kv_len, int n_splits,
                                long long o_split_stride, long long lse_split_stride, int window,
                                const int* seg_start, const int* seg_end) {
  TPB_NVTX("tpb_flash_fwd_ex");
  if (B <= 0 || Tq <= 0 || Hq <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || Tk <= 0) return -2;
  if ((q_tok | q_head | q_batch | k_tok | k_head | k_batch | v_tok | v_head | v_batch | o_tok |
       o_head | o_batch) % 8)
    return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(o)) & 15)
    return -2;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_tmap_bthd(&tq, q, B, Tq, Hq, D, q_tok, q_head, q_batch, kBlockQ))) return r;
  if ((r = make_tmap_bthd(&tk, k, B, Tk, Hkv, D, k_tok, k_head, k_batch, kBlockKV))) return r;
  if ((r = make_tmap_bthd(&tv, v, B, Tk, Hkv, D, v_tok, v_head, v_batch, kBlockKV))) return r;
  AttnFwdParams p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.kv_offset = Tk - Tq;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.O = (__nv_bfloat16*)o; p.o_tok_stride = o_tok; p.o_head_stride = o_head;
  p.o_batch_stride = o_batch; p.lse = lse; p.lse_stride = lse_stride > 0 ? lse_stride : Tq; p.status = status; p.wait_ns = kDefaultWaitNs; p.kv_len = kv_len;
  p.n_splits = n_splits > 1 ? n_splits : 1;
  {
    const int blocks = (Tk + kBlockKV - 1) / kBlockKV;
    p.blocks_per_split = (blocks + p.n_splits - 1) / p.n_splits;
  }
  p.o_split_stride = o_split_stride; p.lse_split_stride = lse_split_stride;
  p.trace = g_fwd_trace; p.trace_cap = g_fwd_trace_cap;
  p.window = window > 0 ? window : 0; p.seg_start = seg_start; p.seg_end = seg_end;
  if (p.n_splits > 1 && causal) return -3;  // splitting is for decode (one query tile, no causal mask)
  if (D == 128) {
    switch (g_fwd_npoly) {
      case 2: return launch_fwd<128, 2>(tq, tk, tv, p, (cudaStream_t)stream);
      case 1: return launch_fwd<128, 1>(tq, tk, tv, p, (cudaStream_t)stream);
      default: return launch_fwd<128, 0>(tq, tk, tv, p, (cudaStream_t)stream);
    }
  }
  // head_dim 64 halves the tensor work per score, so the exponentials dominate: more of them
  // go to the FMA pipe
  return launch_fwd<64, 2>(tq, tk, tv, p, (cudaStream_t)stream);
}

extern "C" int tpb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                             int B, int Tq, int Tk, int Hq, int Hkv, int D, long long q_tok,
                             long long q_head, long long q_batch, long long k_tok,
                             long long k_head, long long k_batch, long long v_tok,
                             long long v_head, long long v_batch, long long o_tok,
                             long long o_head, long long o_batch, int lse_stride, int causal,
                             float scale, uint32_t* status, void* stream, const int* kv_len, int n_splits,
                             long long o_split_stride, long long lse_split_stride) {
  TPB_NVTX("tpb_flash_fwd");
  return tpb_flash_fwd_ex(q, k, v, o, lse, B, Tq, Tk, Hq, Hkv, D, q_tok, q_head, q_batch, k_tok, k_head, k_batch,
                          v_tok, v_head, v_batch, o_tok, o_head, o_batch, lse_stride, causal, scale, status, stream,
                          kv_len, n_splits, o_split_stride, lse_split_stride, 0, nullptr, nullptr);
}

// Share of the exponentials that the forward computes with the polynomial on the FMA pipe instead of
// the special-function unit, for head_dim 128: n of every 4 column pairs (0, 1 or 2).
extern "C" int tpb_flash_fwd_config(int npoly_of_4) {
  if (npoly_of_4 < 0 || npoly_of_4 > 2) return -2;
  g_fwd_npoly = npoly_of_4;
  return 0;
}

// Merge the partials of a split-KV forward (see tpb_flash_fwd): part [n_splits][B, T, H, D] bf16
// contiguous, lse_part [n_splits][B, H, lse_stride]; out by strides, lse_out [B, H, lse_stride] or null.
extern "C" int tpb_attn_split_merge(const void* part, const float* lse_part, void* out, float* lse_out,
                                    int n_splits, int B, int T, int H, int D, long long part_split_stride,
                                    long long lse_split_stride, int lse_stride, long long o_tok,
                                    long long o_head, long long o_batch, void* stream) {
  TPB_NVTX("tpb_attn_split_merge");
  if (B <= 0 || T <= 0 || H <= 0 || n_splits <= 0) return 0;
  if (D & 1) return -1;
  const long long warps = (long long)B * T * H;
  const int grid = (int)((warps * 32 + 255) / 256);
  attn_split_merge_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(part), lse_part, static_cast<__nv_bfloat16*>(out), lse_out, n_splits, B, T,
      H, D, part_split_stride, lse_split_stride, lse_stride, o_tok, o_head, o_batch);
  return (int)cudaGetLastError();
}
