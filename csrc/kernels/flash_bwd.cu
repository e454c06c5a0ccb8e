// Flash attention backward for sm_100a (tcgen05 / TMEM / TMA), GQA-native, causal or full.
//
// Two passes over the recomputed probabilities, each a warp-specialised kernel built from one
// template:
//   * dKV pass: a CTA owns 128 keys of one KV head, keeps K and V in shared memory and streams
//     64-query tiles of Q and dO of every query head of the group; it accumulates
//     dV += P^T dO and dK += dS^T Q in TMEM, so the GQA reduction over the query heads of a
//     group happens inside the accumulator (no expanded K/V, no atomics).
//   * dQ pass: a CTA owns 128 queries of one query head, keeps Q and dO resident and streams
//     64-key tiles of K and V; dQ += dS K in TMEM (deterministic, no atomics).
// Per streamed tile: S = X0 Y0^T and dP = X1 Y1^T (tcgen05.mma, TMEM double-buffered), the four
// "softmax" warps turn them into P and dS = P (dP - delta) * scale, write them as bf16 into
// 128-byte-swizzled tiles, and the accumulating MMAs read those tiles.
//
// Counterpart in the reference: FlashAttention-2 sm80 backward
// (p10/src/backend/cuda/transformers/AttentionKernels.cu:2286-2543), which has no GQA path
// (:2459-2461) and accumulates dQ with fp32 atomics.
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {

int make_tmap_bthd(CUtensorMap* out, const void* base, int B, int T, int H, int D,
                   long long tok_stride, long long head_stride, long long batch_stride, int rows);

constexpr int kBwdThreads = 320;  // TMA warp, MMA warp, 8 P/dS warps (two per TMEM lane quarter)
constexpr int kSoftThreads = 256;
constexpr int kStat = 128;   // rows of the stationary tiles
constexpr int kStream = 64;  // rows of the streamed tiles
constexpr int kYStages = 4;  // streamed-tile ring: loads run three tiles ahead of the MMAs

struct AttnBwdParams {
  int B, Tq, Tk, Hq, Hkv;
  int causal, kv_offset;
  // optional key bounds of a query, as in the forward: window > 0 = local attention; seg_start / seg_end
  // [B * Tq] = keys [start, end) of every query, which with Tq == Tk (packed self-attention, the only form
  // that takes them) are also the queries [start, end) of every key
  int window;
  const int* seg_start;
  const int* seg_end;
  float scale, scale_log2e;
  const float* lse;    // [B, Hq, lse_stride]
  const float* delta;  // [B, Hq, lse_stride]
  int lse_stride;
  __nv_bfloat16* out0;  // dKV: dV ; dQ: unused
  __nv_bfloat16* out1;  // dKV: dK ; dQ: dQ
  long long out_tok, out_head, out_batch;
  uint32_t* status;
  unsigned long long wait_ns;
  unsigned long long* trace;  // optional: timestamps of CTA (0,0,0), see tpb_flash_bwd_set_trace
  int trace_cap;
};

// Debug aid: records (role, iteration, phase, globaltimer) tuples of block (0,0,0).
__device__ __forceinline__ void trace_pt(const AttnBwdParams& p, int role, int it, int phase) {
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
    unsigned long long idx = atomicAdd(p.trace, 1ull);
    if ((int)idx < p.trace_cap) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
      p.trace[1 + idx * 2] = ((unsigned long long)role << 48) | ((unsigned long long)(it & 0xffffff) << 16) | (unsigned)phase;
      p.trace[2 + idx * 2] = t;
    }
  }
}

__device__ __forceinline__ float bwd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));  // pure: let the compiler schedule it
  return y;
}

template <int D>
struct BwdSmem {
  static constexpr int kChunks = D / 64;
  static constexpr int kStatBytes = kStat * D * 2;      // one stationary tile
  static constexpr int kStreamBytes = kStream * D * 2;  // one streamed tile
  static constexpr int kX0 = 0;
  static constexpr int kX1 = kX0 + kStatBytes;
  static constexpr int kY = kX1 + kStatBytes;  // kYStages x (Y0, Y1)
  static constexpr int kStats = kY + 2 * kYStages * kStreamBytes;  // per Y stage: lse[64] then delta[64] (fp32)
  static constexpr int kBar = kStats + kYStages * 2 * kStream * 4;
  static constexpr int kTotal = kBar + 256 + 1024;
  static_assert(kTotal <= 227 * 1024, "attention backward exceeds the shared memory of one CTA");
};

// P = exp2(S * scale_log2e - lse2) and dS = P * (dP * scale - delta * scale) for 32 columns of
// one row, packed to bf16 pairs. Straight-line code: the masked variant selects, it never branches.
//   DKV: per-column statistics (lse, delta of the streamed queries) come from shared memory;
//   dQ : the row's own statistics (already scaled) are in registers.
template <bool DKV, bool MASKED>
__device__ __forceinline__ void pds_math(const uint32_t (&sr)[32], const uint32_t (&dr)[32],
                                         uint32_t stats_sa, float lse2_row, float dsc_row, int y0i,
                                         int y_lo, int y_hi, float scale_log2e, float scale,
                                         uint32_t (&pw)[16], uint32_t (&dw)[16]) {
  constexpr float kLog2e = 1.4426950408889634f;
#pragma unroll
  for (int c = 0; c < 32; c += 4) {
    float l4[4], d4[4];
    if (DKV) {
      float4 a, d;
      asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w) : "r"(stats_sa + c * 4));
      asm("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(d.x), "=f"(d.y), "=f"(d.z), "=f"(d.w) : "r"(stats_sa + (kStream + c) * 4));
      l4[0] = a.x * kLog2e; l4[1] = a.y * kLog2e; l4[2] = a.z * kLog2e; l4[3] = a.w * kLog2e;
      d4[0] = d.x * scale; d4[1] = d.y * scale; d4[2] = d.z * scale; d4[3] = d.w * scale;
    } else {
      l4[0] = l4[1] = l4[2] = l4[3] = lse2_row;
      d4[0] = d4[1] = d4[2] = d4[3] = dsc_row;
    }
    float pr[4], ds[4];
    const float2 sc2 = make_float2(scale_log2e, scale_log2e), s2 = make_float2(scale, scale);
#pragma unroll
    for (int i = 0; i < 4; i += 2) {
      // packed fp32x2 arithmetic: two elements per FMA / MUL
      const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[c + i]), __uint_as_float(sr[c + i + 1])), sc2,
                                  make_float2(-l4[i], -l4[i + 1]));
      const float2 t = __ffma2_rn(make_float2(__uint_as_float(dr[c + i]), __uint_as_float(dr[c + i + 1])), s2,
                                  make_float2(-d4[i], -d4[i + 1]));
      float2 e = make_float2(bwd_exp2(x.x), bwd_exp2(x.y));
      float2 g = __fmul2_rn(e, t);
      if (MASKED) {
        const int yi = y0i + c + i;
        const bool v0 = (yi >= y_lo) & (yi < y_hi), v1 = (yi + 1 >= y_lo) & (yi + 1 < y_hi);
        e.x = v0 ? e.x : 0.f; g.x = v0 ? g.x : 0.f;
        e.y = v1 ? e.y : 0.f; g.y = v1 ? g.y : 0.f;
      }
      pr[i] = e.x; pr[i + 1] = e.y;
      ds[i] = g.x; ds[i + 1] = g.y;
    }
    __nv_bfloat162 p0 = __floats2bfloat162_rn(pr[0], pr[1]), p1 = __floats2bfloat162_rn(pr[2], pr[3]);
    __nv_bfloat162 s0 = __floats2bfloat162_rn(ds[0], ds[1]), s1 = __floats2bfloat162_rn(ds[2], ds[3]);
    pw[c / 2] = *reinterpret_cast<uint32_t*>(&p0);
    pw[c / 2 + 1] = *reinterpret_cast<uint32_t*>(&p1);
    dw[c / 2] = *reinterpret_cast<uint32_t*>(&s0);
    dw[c / 2 + 1] = *reinterpret_cast<uint32_t*>(&s1);
  }
}

// DKV = true : X = (K, V) stationary, Y = (Q, dO) streamed, rows are keys, columns queries.
// DKV = false: X = (Q, dO) stationary, Y = (K, V) streamed, rows are queries, columns keys.
template <int D, bool DKV>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmX1,
                 const __grid_constant__ CUtensorMap tmY0, const __grid_constant__ CUtensorMap tmY1,
                 const AttnBwdParams p) {
  using L = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* x_full = bars;                        // 1
  uint64_t* y_full = bars + 1;                    // kYStages
  uint64_t* y_empty = y_full + kYStages;          // kYStages
  uint64_t* sdp_full = y_empty + kYStages;        // 2
  uint64_t* pds_full = sdp_full + 2;              // 1 (256 arrivals)
  uint64_t* acc_done = pds_full + 1;              // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  volatile uint32_t* abort_w = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  // CTAs start in the order of their linear index; with a causal mask the tile index is the slowest
  // coordinate, heaviest tile first (key tile 0 for dK/dV, the last query tile for dQ), heads and
  // batches the fastest, so that the light CTAs of all heads fill the tail.
  int b = blockIdx.z;
  int hx = blockIdx.y;  // DKV: kv head ; dQ: query head
  int xi = blockIdx.x;
  if (p.causal) {
    const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
    const int hb = gridDim.y * gridDim.z;
    xi = lin / hb;
    hx = (lin % hb) % gridDim.y;
    b = (lin % hb) / gridDim.y;
  }
  const int xb = (DKV || !p.causal) ? xi : (gridDim.x - 1 - xi);
  const int x0 = xb * kStat;  // first key (DKV) or first query (dQ) of this CTA

  // iteration space over streamed tiles
  int y_first = 0, y_count, n_it;
  const long long seg_base = (long long)b * p.Tq;
  if (DKV) {
    // queries of this key tile: from the first key's lower bound to the last key's upper bound
    int q_hi = p.Tq;
    const int k_last = min(x0 + kStat - 1, p.Tk - 1);
    if (p.causal) {
      int qmin = x0 - p.kv_offset;
      y_first = qmin > 0 ? qmin / kStream : 0;
    }
    if (p.window > 0) q_hi = min(q_hi, k_last - p.kv_offset + p.window);
    if (p.seg_start && x0 < p.Tk) y_first = max(y_first, p.seg_start[seg_base + x0] / kStream);
    if (p.seg_end && x0 < p.Tk) q_hi = min(q_hi, p.seg_end[seg_base + k_last]);
    const int nqb = (max(q_hi, 0) + kStream - 1) / kStream;
    y_count = nqb - y_first;
    if (y_count < 0) y_count = 0;
    n_it = y_count * G;
  } else {
    // keys of this query tile: from the first query's lower bound to the last query's upper bound
    int nkb = (p.Tk + kStream - 1) / kStream;
    const int q_last = min(x0 + kStat - 1, p.Tq - 1);
    if (p.causal) {
      int last_key = x0 + kStat - 1 + p.kv_offset;
      int lim = last_key < 0 ? 0 : last_key / kStream + 1;
      nkb = min(nkb, lim);
    }
    if (p.seg_end && x0 < p.Tq) nkb = min(nkb, (p.seg_end[seg_base + q_last] + kStream - 1) / kStream);
    int lo_first = 0;
    if (p.window > 0) lo_first = max(lo_first, x0 + p.kv_offset - p.window + 1);
    if (p.seg_start && x0 < p.Tq) lo_first = max(lo_first, p.seg_start[seg_base + x0]);
    y_first = lo_first / kStream;
    y_count = max(nkb - y_first, 0);
    n_it = y_count;
  }

  if (threadIdx.x == 0) {
    *abort_w = 0;
    mbar_init(x_full, 1);
    for (int i = 0; i < kYStages; ++i) {
      mbar_init(&y_full[i], 1);
      mbar_init(&y_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
    }
    mbar_init(pds_full, kSoftThreads);
    mbar_init(acc_done, 1);
    fence_barrier_init();
    prefetch_tmap(&tmX0);
    prefetch_tmap(&tmX1);
    prefetch_tmap(&tmY0);
    prefetch_tmap(&tmY1);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc0 = tmem_base + 256;
  const uint32_t tmem_acc1 = tmem_base + 384;
  WaitCtx wc{abort_w, p.status, p.wait_ns};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_it > 0) {
      mbar_arrive_expect_tx(x_full, 2 * L::kStatBytes);
      // DKV: X tiles are K/V of kv head hx ; dQ: X tiles are Q/dO of query head hx
#pragma unroll
      for (int c = 0; c < L::kChunks; ++c) {
        tma_load_4d(smem + L::kX0 + c * (kStat * 128), &tmX0, x_full, c * 64, hx, x0, b);
        tma_load_4d(smem + L::kX1 + c * (kStat * 128), &tmX1, x_full, c * 64, hx, x0, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int s = it % kYStages;
        const uint32_t ph = (it / kYStages) & 1;
        if (!mbar_wait_relaxed(&y_empty[s], ph ^ 1, wc, 1)) break;
        trace_pt(p, 0, it, 1);
        int hy, yb;
        if (DKV) { hy = hx * G + it / y_count; yb = y_first + it % y_count; }
        else { hy = hx / G; yb = y_first + it; }
        uint8_t* y0 = smem + L::kY + s * 2 * L::kStreamBytes;
        uint8_t* y1 = y0 + L::kStreamBytes;
        mbar_arrive_expect_tx(&y_full[s], 2 * L::kStreamBytes + (DKV ? 2 * kStream * 4 : 0));
        if (DKV) {
          // the per-query statistics of the streamed tile ride along with it
          const long long so = ((long long)b * p.Hq + hy) * p.lse_stride + (long long)yb * kStream;
          float* st = reinterpret_cast<float*>(smem + L::kStats) + s * 2 * kStream;
          bulk_load_1d(st, p.lse + so, kStream * 4, &y_full[s]);
          bulk_load_1d(st + kStream, p.delta + so, kStream * 4, &y_full[s]);
        }
#pragma unroll
        for (int c = 0; c < L::kChunks; ++c) {
          tma_load_4d(y0 + c * (kStream * 128), &tmY0, &y_full[s], c * 64, hy, yb * kStream, b);
          tma_load_4d(y1 + c * (kStream * 128), &tmY1, &y_full[s], c * 64, hy, yb * kStream, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop with uniform control flow and an elected lane issues: tcgen05
    // operands live in uniform registers, and a divergent `if (lane == 0)` region would move every
    // one of them there per instruction, which costs more than a 128 x 64 x 16 MMA takes to run.
    if (n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(kStat, kStream, 1, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_f16(kStat, D, 1, 0, 1);
      constexpr uint32_t hi = smem_desc_hi(1024);
      const uint32_t x0_lo = smem_desc_lo(smem_u32(smem + L::kX0), 16);
      const uint32_t x1_lo = smem_desc_lo(smem_u32(smem + L::kX1), 16);
      const uint32_t yk_lo = smem_desc_lo(smem_u32(smem + L::kY), 16);               // streamed tiles, K-major view
      const uint32_t ym_lo = smem_desc_lo(smem_u32(smem + L::kY), kStream * 128);    // the same tiles, MN-major view
      auto issue_sdp = [&](int it) -> bool {
        const int ys = it % kYStages;
        const uint32_t yph = (it / kYStages) & 1;
        const int s = it & 1;
        if (!mbar_wait_warp(&y_full[ys], yph, wc, 2)) return false;
        if (lane == 0) trace_pt(p, 1, it, 1);
        // Slot s last held iteration it - 2: its S / dP were read by the P/dS warps before they
        // arrived on pds_full(it - 2), and its P / dS (same columns) are consumed by MMAs issued
        // earlier by this warp, which the tensor pipe executes in order before these.
        tc_fence_after_sync();
        const uint32_t y0_lo = yk_lo + ys * ((2 * L::kStreamBytes) >> 4);
        const uint32_t y1_lo = y0_lo + (L::kStreamBytes >> 4);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xo = ((kk / 4) * (kStat * 128) + (kk % 4) * 32) >> 4;
            const uint32_t yo = ((kk / 4) * (kStream * 128) + (kk % 4) * 32) >> 4;
            umma_f16_ss_w(tmem_base + s * 128, x0_lo + xo, hi, y0_lo + yo, hi, idesc_s, kk != 0);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t xo = ((kk / 4) * (kStat * 128) + (kk % 4) * 32) >> 4;
            const uint32_t yo = ((kk / 4) * (kStream * 128) + (kk % 4) * 32) >> 4;
            umma_f16_ss_w(tmem_base + s * 128 + 64, x1_lo + xo, hi, y1_lo + yo, hi, idesc_s, kk != 0);
          }
          umma_commit(&sdp_full[s]);
        }
        __syncwarp();
        return true;
      };
      bool ok = mbar_wait_warp(x_full, 0, wc, 4);
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) {
          if (!issue_sdp(it + 1)) break;
        }
        const int s = it % kYStages;
        if (!mbar_wait_warp(pds_full, it & 1, wc, 5)) break;
        if (lane == 0) trace_pt(p, 1, it, 3);
        tc_fence_after_sync();
        const uint32_t y0_lo = ym_lo + s * ((2 * L::kStreamBytes) >> 4);
        const uint32_t y1_lo = y0_lo + (L::kStreamBytes >> 4);
        // P and dS are the A operands straight from TMEM: bf16 pairs written over the S / dP
        // columns; k-step kk (16 streamed rows) sits at column (kk / 2) * 32 + (kk % 2) * 8
        const uint32_t t_p = tmem_base + (it & 1) * 128;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < kStream / 16; ++kk) {
            const uint32_t a_col = (kk >> 1) * 32 + (kk & 1) * 8;
            // acc1 += dS * Y0  (dK += dS^T Q  or  dQ += dS K)
            umma_f16_ts_w(tmem_acc1, t_p + 64 + a_col, y0_lo + kk * (2048 >> 4), hi, idesc_acc, (it | kk) != 0);
            if (DKV) {
              // acc0 += P^T * dO
              umma_f16_ts_w(tmem_acc0, t_p + a_col, y1_lo + kk * (2048 >> 4), hi, idesc_acc, (it | kk) != 0);
            }
          }
          umma_commit(&y_empty[s]);
          if (it == n_it - 1) umma_commit(acc_done);
        }
        __syncwarp();
        if (lane == 0) trace_pt(p, 1, it, 4);
      }
    }
  } else {
    // ---------------------------------------------------------------- P / dS warps
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;  // which 32 of the tile's 64 columns this warp handles
    const int row = qd * 32 + lane;
    const int xi = x0 + row;  // key index (DKV) or query index (dQ)
    const uint32_t t_lane = ((uint32_t)(qd * 32) << 16);
    const float log2e = 1.4426950408889634f;
    float lse_row = 0.f, delta_row = 0.f;
    if (!DKV) {
      if (xi < p.Tq) {
        long long o = ((long long)b * p.Hq + hx) * p.lse_stride + xi;
        lse_row = p.lse[o];
        delta_row = p.delta[o];
      }
    }
    // streamed indices (queries for dKV, keys for dQ) that this row may pair with
    int y_lo, y_hi;
    if (DKV) {
      y_lo = (xi < p.Tk) ? (p.causal ? max(xi - p.kv_offset, 0) : 0) : 0x3fffffff;
      y_hi = p.Tq;
      if (p.window > 0) y_hi = min(y_hi, xi - p.kv_offset + p.window);
      if (xi < p.Tk) {
        if (p.seg_start) y_lo = max(y_lo, p.seg_start[seg_base + xi]);
        if (p.seg_end) y_hi = min(y_hi, p.seg_end[seg_base + xi]);
      }
    } else {
      y_lo = 0;
      y_hi = (xi < p.Tq) ? (p.causal ? min(p.Tk, xi + p.kv_offset + 1) : p.Tk) : 0;
      if (p.window > 0) y_lo = max(y_lo, xi + p.kv_offset - p.window + 1);
      if (xi < p.Tq) {
        if (p.seg_start) y_lo = max(y_lo, p.seg_start[seg_base + xi]);
        if (p.seg_end) y_hi = min(y_hi, p.seg_end[seg_base + xi]);
      }
    }
    lse_row *= log2e;
    delta_row *= p.scale;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      int yb;
      if (DKV) yb = y_first + it % y_count;
      else yb = y_first + it;
      const int y0i = yb * kStream + half * 32;  // first query (DKV) or key (dQ) of this warp's columns
      if (!mbar_wait_warp(&sdp_full[s], ph, wc, 6)) { ok = false; break; }
      if (threadIdx.x == 64) trace_pt(p, 2, it, 1);
      tc_fence_after_sync();
      uint32_t sr[32], dr[32];
      tmem_ld_32x32b_x32(tmem_base + t_lane + s * 128 + half * 32, sr);
      tmem_ld_32x32b_x32(tmem_base + t_lane + s * 128 + 64 + half * 32, dr);
      tmem_ld_wait();
      if (threadIdx.x == 64) trace_pt(p, 2, it, 2);

      // Valid streamed indices of this thread's row form one interval [lo, hi): tiles that lie
      // entirely inside it take the predicate-free path (warp-uniform choice).
      const bool need_mask = __any_sync(0xffffffffu, (y0i < y_lo) || (y0i + 32 > y_hi));
      uint32_t lse_sa = 0;
      if (DKV) {
        // statistics landed with the tile (the wait below returns at once and orders the read)
        const int ys = it % kYStages;
        if (!mbar_wait_warp(&y_full[ys], (it / kYStages) & 1, wc, 9)) { ok = false; break; }
        lse_sa = smem_u32(smem + L::kStats) + (ys * 2 * kStream + half * 32) * 4;
      }
      uint32_t pw[16], dw[16];
      if (need_mask) pds_math<DKV, true>(sr, dr, lse_sa, lse_row, delta_row, y0i, y_lo, y_hi, p.scale_log2e, p.scale, pw, dw);
      else pds_math<DKV, false>(sr, dr, lse_sa, lse_row, delta_row, y0i, y_lo, y_hi, p.scale_log2e, p.scale, pw, dw);
      if (threadIdx.x == 64) trace_pt(p, 2, it, 3);
      // P / dS (bf16 pairs) go back into this warp's own S / dP columns
      if (DKV) tmem_st_32x32b_x16(tmem_base + t_lane + s * 128 + half * 32, pw);
      tmem_st_32x32b_x16(tmem_base + t_lane + s * 128 + 64 + half * 32, dw);
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(pds_full);
      if (threadIdx.x == 64) trace_pt(p, 2, it, 5);
    }
    if (ok && n_it > 0) ok = mbar_wait_warp(acc_done, 0, wc, 8);
    if (ok) {
      tc_fence_after_sync();
      const int t_lim = DKV ? p.Tk : p.Tq;
      const long long obase = (long long)b * p.out_batch + (long long)xi * p.out_tok +
                              (long long)hx * p.out_head;
#pragma unroll 1
      for (int a = DKV ? 0 : 1; a < 2; ++a) {
        __nv_bfloat16* orow = (a == 0 ? p.out0 : p.out1) + obase;
        const uint32_t t_acc = (a == 0 ? tmem_acc0 : tmem_acc1) + t_lane;
#pragma unroll 1
        for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
          uint32_t o[32];
          if (n_it > 0) {
            tmem_ld_32x32b_x32(t_acc + c * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0;
          }
          if (xi < t_lim) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 v;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(__uint_as_float(o[g * 8 + 0]),
                                                        __uint_as_float(o[g * 8 + 1]));
              __nv_bfloat162 t1 = __floats2bfloat162_rn(__uint_as_float(o[g * 8 + 2]),
                                                        __uint_as_float(o[g * 8 + 3]));
              __nv_bfloat162 t2 = __floats2bfloat162_rn(__uint_as_float(o[g * 8 + 4]),
                                                        __uint_as_float(o[g * 8 + 5]));
              __nv_bfloat162 t3 = __floats2bfloat162_rn(__uint_as_float(o[g * 8 + 6]),
                                                        __uint_as_float(o[g * 8 + 7]));
              v.x = *reinterpret_cast<uint32_t*>(&t0);
              v.y = *reinterpret_cast<uint32_t*>(&t1);
              v.z = *reinterpret_cast<uint32_t*>(&t2);
              v.w = *reinterpret_cast<uint32_t*>(&t3);
              *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = v;
            }
          }
        }
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
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, t] = sum_d O[b, t, h, d] * dO[b, t, h, d]; one warp per (b, t, h).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ dout, float* __restrict__ delta,
                                  int B, int T, int H, int D, long long o_tok, long long o_head,
                                  long long o_batch, long long d_tok, long long d_head,
                                  long long d_batch, int lse_stride) {
  long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  long long total = (long long)B * T * H;
  if (w >= total) return;
  int h = w % H;
  long long bt = w / H;
  int t = bt % T;
  int b = bt / T;
  const __nv_bfloat16* op = o + b * o_batch + t * o_tok + h * o_head;
  const __nv_bfloat16* dp = dout + b * d_batch + t * d_tok + h * d_head;
  float s = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + i));
    float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + i));
    s += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[((long long)b * H + h) * lse_stride + t] = s;
}

static unsigned long long* g_bwd_trace = nullptr;
static int g_bwd_trace_cap = 0;

template <int D, bool DKV>
static int launch_bwd(const CUtensorMap& x0, const CUtensorMap& x1, const CUtensorMap& y0,
                      const CUtensorMap& y1, const AttnBwdParams& p, dim3 grid,
                      cudaStream_t stream) {
  using L = BwdSmem<D>;
  auto kern = flash_bwd_kernel<D, DKV>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  kern<<<grid, kBwdThreads, L::kTotal, stream>>>(x0, x1, y0, y1, p);
  return (int)cudaGetLastError();
}

}  // namespace tpb

using namespace tpb;

// lse / delta: [B, Hq, lse_stride] fp32 with lse_stride a multiple of 64 and >= Tq rounded up
// to 64 (the dKV pass reads whole 64-query vectors). delta is scratch written here.
// window / seg_start / seg_end as in tpb_flash_fwd_ex; segment bounds need Tq == Tk.
extern "C" int tpb_flash_bwd_ex(const void* dout, const void* q, const void* k, const void* v,
                                const void* o, const float* lse, float* delta, void* dq, void* dk,
                                void* dv, int B, int Tq, int Tk, int Hq, int Hkv, int D,
                                long long q_tok, long long q_head, long long q_batch, long long k_tok,
                                long long k_head, long long k_batch, long long v_tok,
                                long long v_head, long long v_batch, long long o_tok,
                                long long o_head, long long o_batch, long long do_tok,
                                long long do_head, long long do_batch, long long dq_tok,
                                long long dq_head, long long dq_batch, long long dkv_tok,
                                long long dkv_head, long long dkv_batch, int lse_stride, int causal,
                                float scale, uint32_t* status, void* stream_, int window, const int* seg_start,
                                const int* seg_end) {
  TPB_NVTX("tpb_flash_bwd_ex");
  cudaStream_t stream = (cudaStream_t)stream_;
  if (B <= 0 || Tq <= 0 || Hq <= 0) return 0;
  if ((seg_start || seg_end) && Tq != Tk) return -2;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || Tk <= 0) return -2;
  if (lse_stride % 64 || lse_stride < (Tq + 63) / 64 * 64) return -2;
  if ((q_tok | q_head | q_batch | k_tok | k_head | k_batch | v_tok | v_head | v_batch | do_tok |
       do_head | do_batch | dq_tok | dq_head | dq_batch | dkv_tok | dkv_head | dkv_batch) % 8)
    return -2;
  // delta
  {
    long long warps = (long long)B * Tq * Hq;
    long long threads = warps * 32;
    attn_delta_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, B, Tq, Hq, D, o_tok, o_head,
        o_batch, do_tok, do_head, do_batch, lse_stride);
  }
  AttnBwdParams p;
  p.B = B; p.Tq = Tq; p.Tk = Tk; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal;
  p.kv_offset = Tk - Tq; p.scale = scale; p.scale_log2e = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.lse_stride = lse_stride; p.status = status;
  p.wait_ns = kDefaultWaitNs;
  p.trace = g_bwd_trace; p.trace_cap = g_bwd_trace_cap;
  p.window = window > 0 ? window : 0; p.seg_start = seg_start; p.seg_end = seg_end;
  int r;
  // ---- dK / dV: [B, Tk, Hkv, D] by the dkv strides (dk and dv share them)
  {
    CUtensorMap tk, tv, tq, tdo;
    if ((r = make_tmap_bthd(&tk, k, B, Tk, Hkv, D, k_tok, k_head, k_batch, kStat))) return r;
    if ((r = make_tmap_bthd(&tv, v, B, Tk, Hkv, D, v_tok, v_head, v_batch, kStat))) return r;
    if ((r = make_tmap_bthd(&tq, q, B, Tq, Hq, D, q_tok, q_head, q_batch, kStream))) return r;
    if ((r = make_tmap_bthd(&tdo, dout, B, Tq, Hq, D, do_tok, do_head, do_batch, kStream))) return r;
    p.out0 = (__nv_bfloat16*)dv; p.out1 = (__nv_bfloat16*)dk;
    p.out_tok = dkv_tok; p.out_head = dkv_head; p.out_batch = dkv_batch;
    dim3 grid((Tk + kStat - 1) / kStat, Hkv, B);
    r = (D == 128) ? launch_bwd<128, true>(tk, tv, tq, tdo, p, grid, stream)
                   : launch_bwd<64, true>(tk, tv, tq, tdo, p, grid, stream);
    if (r) return r;
  }
  // ---- dQ: [B, Tq, Hq, D] by the dq strides
  {
    CUtensorMap tq, tdo, tk, tv;
    if ((r = make_tmap_bthd(&tq, q, B, Tq, Hq, D, q_tok, q_head, q_batch, kStat))) return r;
    if ((r = make_tmap_bthd(&tdo, dout, B, Tq, Hq, D, do_tok, do_head, do_batch, kStat))) return r;
    if ((r = make_tmap_bthd(&tk, k, B, Tk, Hkv, D, k_tok, k_head, k_batch, kStream))) return r;
    if ((r = make_tmap_bthd(&tv, v, B, Tk, Hkv, D, v_tok, v_head, v_batch, kStream))) return r;
    p.out0 = nullptr; p.out1 = (__nv_bfloat16*)dq;
    p.out_tok = dq_tok; p.out_head = dq_head; p.out_batch = dq_batch;
    dim3 grid((Tq + kStat - 1) / kStat, Hq, B);
    r = (D == 128) ? launch_bwd<128, false>(tq, tdo, tk, tv, p, grid, stream)
                   : launch_bwd<64, false>(tq, tdo, tk, tv, p, grid, stream);
    if (r) return r;
  }
  return 0;
}

// Debug aid: buf = device array of 1 + 2 * cap uint64 (buf[0] = record count, zero it first). The
// next backward launches record role / iteration / phase timestamps of block (0,0,0) of BOTH
// passes into it. Pass null to switch tracing off.
extern "C" int tpb_flash_bwd(const void* dout, const void* q, const void* k, const void* v,
                             const void* o, const float* lse, float* delta, void* dq, void* dk,
                             void* dv, int B, int Tq, int Tk, int Hq, int Hkv, int D,
                             long long q_tok, long long q_head, long long q_batch, long long k_tok,
                             long long k_head, long long k_batch, long long v_tok,
                             long long v_head, long long v_batch, long long o_tok,
                             long long o_head, long long o_batch, long long do_tok,
                             long long do_head, long long do_batch, long long dq_tok,
                             long long dq_head, long long dq_batch, long long dkv_tok,
                             long long dkv_head, long long dkv_batch, int lse_stride, int causal,
                             float scale, uint32_t* status, void* stream_) {
  TPB_NVTX("tpb_flash_bwd");
  return tpb_flash_bwd_ex(dout, q, k, v, o, lse, delta, dq, dk, dv, B, Tq, Tk, Hq, Hkv, D, q_tok, q_head, q_batch,
                          k_tok, k_head, k_batch, v_tok, v_head, v_batch, o_tok, o_head, o_batch, do_tok, do_head,
                          do_batch, dq_tok, dq_head, dq_batch, dkv_tok, dkv_head, dkv_batch, lse_stride, causal, scale,
                          status, stream_, 0, nullptr, nullptr);
}

extern "C" int tpb_flash_bwd_set_trace(unsigned long long* buf, int cap) {
  tpb::g_bwd_trace = buf;
  tpb::g_bwd_trace_cap = cap;
  return 0;
}
