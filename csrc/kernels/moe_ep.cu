// Expert-parallel MoE token exchange over NVLink peer memory (dropless, no host sync).
//
//   route    : histogram of the local (token, k) -> expert assignments; the histogram is pushed
//              into every peer's table; once all tables arrived every rank derives - identically -
//              the layout of every destination buffer (expert segments padded to 128 rows, one
//              sub-range per source rank) and gives each local assignment its destination row.
//   dispatch : each assignment's token row is stored straight into the owning rank's expert
//              buffer at its final, expert-sorted position (the permutation IS the transfer),
//              optionally scaled (the backward of combine).
//   combine  : each token pulls its k expert outputs from the owners' buffers and sums them with
//              the gating weights in fp32; optionally also returns the k dot products
//              <g[t], y[row]> needed for the gate-weight gradient.
// Every cross-rank wait is a bounded poll of local memory; overflow of the destination buffer is
// reported through the status word and the surplus assignments are dropped (row = -1).
//
// The reference has no device path for this: TokenSwitch is a single-process Python row-copy loop
// (tensorplay/distributed/_token_switch.py:85-140).
#include "sm100.cuh"
#include "tpb_api.h"

#include <string.h>

namespace tpb {

constexpr int kMoeMaxExperts = 1024;
constexpr int kMoeMaxRanks = 16;

struct MoeSync {
  uint32_t* pad_local;
  uint32_t* pad_peer[kMoeMaxRanks];
  int world, rank;
  uint32_t epoch;
  unsigned long long wait_ns;
  uint32_t* status;
};

__device__ __forceinline__ uint4 moe_ld_peer(const void* ptr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr)
               : "memory");
  return v;
}

// One CTA of 1024 threads.
//   topk_idx [n_assign] int32 expert ids (n_assign = tokens * k)
//   counts_tbl: symmetric [world, E] int32; row s is written by rank s on every rank
//   outputs: dst_rank[n_assign], dst_row[n_assign] (row -1 = dropped),
//            offs_local[E_local + 1] padded expert offsets of THIS rank's buffer, followed by
//            E_local entries: the first padding row of each local expert's segment (the rows from
//            there to the next offset hold no token; moe_zero_pad_kernel clears them),
//            recv_rows (device scalar) = rows in use on this rank (padded).
__global__ void __launch_bounds__(1024)
moe_route_kernel(const int* __restrict__ topk_idx, int n_assign, int E, int E_local,
                 int* const* counts_tbl_peer /* [world] pointers to each rank's table */,
                 int* __restrict__ counts_tbl_local, int* __restrict__ dst_rank,
                 int* __restrict__ dst_row, int* __restrict__ offs_local, int* __restrict__ recv_rows,
                 char* __restrict__ zero_buf, int zero_row_bytes, int cap_rows, MoeSync s,
                 int ready_slot) {
  __shared__ int hist[kMoeMaxExperts];
  __shared__ int base[kMoeMaxExperts];    // first destination row of MY tokens for expert e
  __shared__ int cursor[kMoeMaxExperts];
  __shared__ int seg_total[kMoeMaxExperts];  // tokens of all ranks for expert e
  __shared__ int ok_sh, overflow_sh;
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) { hist[e] = 0; cursor[e] = 0; }
  if (tid == 0) { ok_sh = 1; overflow_sh = 0; }
  __syncthreads();
  for (int a = tid; a < n_assign; a += blockDim.x) {
    int e = topk_idx[a];
    if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  // push my histogram row into every rank's table (own included)
  for (int r = 0; r < s.world; ++r) {
    int* row = counts_tbl_peer[r] + (size_t)s.rank * E;
    for (int e = tid; e < E; e += blockDim.x) row[e] = hist[e];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < s.world) st_release_sys(s.pad_peer[tid] + ready_slot + s.rank, s.epoch);
  if (tid < s.world) {
    if (!flag_wait_ge(s.pad_local + ready_slot + tid, s.epoch, true, s.status, s.wait_ns, 30)) ok_sh = 0;
  }
  __syncthreads();
  if (!ok_sh) {
    for (int a = tid; a < n_assign; a += blockDim.x) { dst_row[a] = -1; dst_rank[a] = 0; }
    for (int j = tid; j < 2 * E_local + 1; j += blockDim.x) offs_local[j] = 0;
    if (tid == 0) *recv_rows = 0;
    return;
  }
  // per expert: total over ranks and my sub-offset inside the segment
  for (int e = tid; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int r = 0; r < s.world; ++r) {
      int c = *reinterpret_cast<volatile int*>(counts_tbl_local + (size_t)r * E + e);
      if (r < s.rank) before += c;
      tot += c;
    }
    seg_total[e] = tot;
    base[e] = before;  // completed below with the expert's segment start
  }
  __syncthreads();
  // segment starts per destination rank (padded to 128): one thread per destination rank
  if (tid < s.world) {
    int row = 0;
    for (int j = 0; j < E_local; ++j) {
      const int e = tid * E_local + j;
      if (tid == s.rank) offs_local[j] = row;
      base[e] += row;
      row += (seg_total[e] + 127) / 128 * 128;
    }
    if (tid == s.rank) {
      offs_local[E_local] = row;
      *recv_rows = row;
    }
    if (row > cap_rows) overflow_sh = 1;
  }
  __syncthreads();
  if (overflow_sh) {
    if (tid == 0 && s.status) atomicCAS(s.status, 0u, kStatusBadArgs | (31u << 8));
    for (int a = tid; a < n_assign; a += blockDim.x) { dst_row[a] = -1; dst_rank[a] = 0; }
    for (int j = tid; j < 2 * E_local + 1; j += blockDim.x) offs_local[j] = 0;
    if (tid == 0) *recv_rows = 0;
    return;
  }
  // destination row of every assignment
  for (int a = tid; a < n_assign; a += blockDim.x) {
    int e = topk_idx[a];
    if (e >= 0 && e < E) {
      dst_rank[a] = e / E_local;
      dst_row[a] = base[e] + atomicAdd(&cursor[e], 1);
    } else {
      dst_rank[a] = 0;
      dst_row[a] = -1;
    }
  }
  // first padding row of each of my expert segments (nobody writes those rows)
  for (int j = tid; j < E_local; j += blockDim.x)
    offs_local[E_local + 1 + j] = offs_local[j] + seg_total[s.rank * E_local + j];
}

// Clears the padding rows of this rank's expert buffer: CTA (j, c) takes a share of expert j's rows
// [pad_begin[j], offs[j + 1]) (at most 127 rows).
__global__ void __launch_bounds__(256)
moe_zero_pad_kernel(const int* __restrict__ offs, int E_local, char* __restrict__ buf, int row_bytes) {
  const int j = blockIdx.x;
  const int r0 = offs[E_local + 1 + j], r1 = offs[j + 1];
  const long long nvec = (long long)max(r1 - r0, 0) * row_bytes / 16;
  uint4* z = reinterpret_cast<uint4*>(buf + (long long)r0 * row_bytes);
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.y * blockDim.x)
    z[i] = make_uint4(0, 0, 0, 0);
}

struct MoePeerBufs {
  char* p[kMoeMaxRanks];
};

// Warp per assignment: row of x (H bf16) -> peer buffer row. scale (optional, [n_assign] fp32).
// After the last block every peer is told that this rank's rows have landed (done_slot).
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride, int k, int n_assign,
                    const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                    const float* __restrict__ scale, MoePeerBufs bufs, int H, MoeSync s,
                    int done_slot, uint32_t* block_counter) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (long long a = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); a < n_assign;
       a += (long long)gridDim.x * wpb) {
    const int row = dst_row[a];
    if (row < 0) continue;
    const int t = (int)(a / k);
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * x_stride);
    uint4* dst = reinterpret_cast<uint4*>(bufs.p[dst_rank[a]] + (long long)row * H * 2);
    const float sc = scale ? scale[a] : 1.f;
    for (int v = lane; v < nvec; v += 32) {
      uint4 u = src[v];
      if (scale) {
        __nv_bfloat162* hb = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(hb[j]);
          hb[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      dst[v] = u;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned prev = atomicAdd(block_counter, 1u);
    if (prev == gridDim.x - 1) {
      *block_counter = 0;
      __threadfence_system();
      for (int r = 0; r < s.world; ++r) st_release_sys(s.pad_peer[r] + done_slot + s.rank, s.epoch);
    }
  }
}

// Warp per token: out[t] = sum_k w[t,k] * buf[dst_rank][dst_row] ; w == null means weight 1.
// dots (optional, [tokens * k]): <g[t], row> for the gate-weight gradient (g given instead of out
// accumulation when dots_only).
template <int KB>  // rows of a token requested together: min(8, k rounded up to a power of two)
__global__ void __launch_bounds__(256)
moe_combine_kernel(MoePeerBufs bufs, const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                   const float* __restrict__ w, int k, int tokens, int H,
                   __nv_bfloat16* __restrict__ out, long long out_stride,
                   const __nv_bfloat16* __restrict__ g, long long g_stride, float* __restrict__ dots,
                   MoeSync s, int ready_slot) {
  // expert outputs of every rank must be complete
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (threadIdx.x < s.world) {
    if (!flag_wait_ge(s.pad_local + ready_slot + threadIdx.x, s.epoch, true, s.status, s.wait_ns, 32)) ok_sh = 0;
  }
  __syncthreads();
  if (!ok_sh) return;
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (long long t = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); t < tokens;
       t += (long long)gridDim.x * wpb) {
    // lane kk holds the source row of assignment kk (k0 + kk for k > 32); the k rows of a token are
    // requested together, KB at a time: one NVLink round trip per group instead of one per row
    for (int v0 = lane; v0 < nvec; v0 += 32) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int k0 = 0; k0 < k; k0 += KB) {
        uint4 u[KB];
        float wk[KB];
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) {
          const long long a = t * k + k0 + kk;
          const int row = (k0 + kk < k) ? dst_row[a] : -1;
          wk[kk] = 0.f;
          u[kk] = make_uint4(0, 0, 0, 0);
          if (row >= 0) {
            u[kk] = moe_ld_peer(reinterpret_cast<const uint4*>(bufs.p[dst_rank[a]] + (long long)row * H * 2) + v0);
            wk[kk] = w ? w[a] : 1.f;
          }
        }
#pragma unroll
        for (int kk = 0; kk < KB; ++kk) {
          const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&u[kk]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(hb[j]);
            acc[2 * j] += wk[kk] * f.x;
            acc[2 * j + 1] += wk[kk] * f.y;
          }
        }
      }
      if (out) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        reinterpret_cast<uint4*>(out + t * out_stride)[v0] = o;
      }
    }
    if (dots) {
      for (int kk = 0; kk < k; ++kk) {
        const long long a = t * k + kk;
        const int row = dst_row[a];
        float d = 0.f;
        if (row >= 0) {
          for (int v0 = lane; v0 < nvec; v0 += 32) {
            uint4 u = moe_ld_peer(reinterpret_cast<const uint4*>(bufs.p[dst_rank[a]] + (long long)row * H * 2) + v0);
            uint4 gg = reinterpret_cast<const uint4*>(g + t * g_stride)[v0];
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&u);
            const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gg);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float2 f = __bfloat1622float2(hb[j]);
              float2 q = __bfloat1622float2(gb[j]);
              d += f.x * q.x + f.y * q.y;
            }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) dots[a] = d;
      }
    }
  }
}

// Publish "this rank's expert outputs for `epoch` are complete" to every peer.
__global__ void moe_signal_kernel(MoeSync s, int slot) {
  if (threadIdx.x < s.world) {
    __threadfence_system();
    st_release_sys(s.pad_peer[threadIdx.x] + slot + s.rank, s.epoch);
  }
}

// Warp per row: out[r] = <a[r], b[r]> in fp32, stored as the bf16 pair (hi, lo) with hi + lo == the
// fp32 value to 16 bits, in columns 0 and 1 of an 8-column bf16 row (columns 2..7 zero), so that the
// row-pull kernel above can fetch it like any other expert row. rows_dev: device word with the number
// of rows in use.
__global__ void __launch_bounds__(256)
moe_rowdot_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                  __nv_bfloat16* __restrict__ out, const int* __restrict__ rows_dev, int cap_rows, int H) {
  const int rows = min(*rows_dev, cap_rows);
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    float acc = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 ua = reinterpret_cast<const uint4*>(a + r * H)[v];
      const uint4 ub = reinterpret_cast<const uint4*>(b + r * H)[v];
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&ua);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&ub);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      const __nv_bfloat16 hi = __float2bfloat16(acc);
      const __nv_bfloat16 lo = __float2bfloat16(acc - __bfloat162float(hi));
      uint4 o4 = make_uint4(0, 0, 0, 0);
      __nv_bfloat162 p2 = __halves2bfloat162(hi, lo);
      o4.x = *reinterpret_cast<uint32_t*>(&p2);
      reinterpret_cast<uint4*>(out)[r] = o4;
    }
  }
}

static MoeSync make_moe_sync(const SymmView* sv, size_t pad_off, uint32_t epoch, uint32_t* status,
                             double wait_s) {
  MoeSync s;
  memset(&s, 0, sizeof(s));
  s.world = sv->world;
  s.rank = sv->rank;
  s.pad_local = reinterpret_cast<uint32_t*>(sv->peer[sv->rank] + pad_off);
  for (int r = 0; r < sv->world; ++r) s.pad_peer[r] = reinterpret_cast<uint32_t*>(sv->peer[r] + pad_off);
  s.epoch = epoch;
  s.wait_ns = wait_s > 0 ? (unsigned long long)(wait_s * 1e9) : kDefaultWaitNs;
  s.status = status;
  return s;
}

}  // namespace tpb

using namespace tpb;

// counts_off: arena offset of the [world, E] int32 table; xbuf_off: arena offset of this rank's
// expert input buffer (its padding rows get zeroed by a second, multi-CTA launch), or (size_t)-1.
// offs_local: 2 * E_local + 1 ints (see moe_route_kernel).
// peer_tbl_dev: device array of `world` pointers (filled by the caller once) to each rank's table.
extern "C" int tpb_moe_route(const int* topk_idx, int n_assign, int E, int* const* peer_tbl_dev,
                             size_t counts_off, int* dst_rank, int* dst_row, int* offs_local,
                             int* recv_rows, size_t xbuf_off, int row_bytes, int cap_rows,
                             size_t pad_off, int ready_slot, uint32_t epoch, double wait_s,
                             uint32_t* status, void* stream) {
  TPB_NVTX("tpb_moe_route");
  const SymmView* sv = symm_view();
  if (!sv || E > kMoeMaxExperts || E % sv->world) return -2;
  MoeSync s = make_moe_sync(sv, pad_off, epoch, status, wait_s);
  char* zb = xbuf_off == (size_t)-1 ? nullptr : sv->peer[sv->rank] + xbuf_off;
  moe_route_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(
      topk_idx, n_assign, E, E / sv->world, peer_tbl_dev,
      reinterpret_cast<int*>(sv->peer[sv->rank] + counts_off), dst_rank, dst_row, offs_local,
      recv_rows, zb, row_bytes, cap_rows, s, ready_slot);
  if (zb) moe_zero_pad_kernel<<<dim3(E / sv->world, 4), 256, 0, (cudaStream_t)stream>>>(offs_local, E / sv->world, zb, row_bytes);
  return (int)cudaGetLastError();
}

// Fills a host array with the address of the buffer at arena offset `off` on every rank.
extern "C" int tpb_symm_peer_ptrs(size_t off, void** out, int n) {
  const SymmView* sv = symm_view();
  if (!sv || n < sv->world) return -2;
  for (int r = 0; r < sv->world; ++r) out[r] = sv->peer[r] + off;
  return 0;
}

extern "C" int tpb_moe_dispatch(const void* x, long long x_stride, int k, int n_assign,
                                const int* dst_rank, const int* dst_row, const float* scale,
                                size_t buf_off, int H, size_t pad_off, int done_slot,
                                uint32_t epoch, uint32_t* block_counter, int ctas,
                                uint32_t* status, void* stream) {
  TPB_NVTX("tpb_moe_dispatch");
  const SymmView* sv = symm_view();
  if (!sv || H % 8) return -2;
  MoePeerBufs b;
  memset(&b, 0, sizeof(b));
  for (int r = 0; r < sv->world; ++r) b.p[r] = sv->peer[r] + buf_off;
  MoeSync s = make_moe_sync(sv, pad_off, epoch, status, 0);
  int grid = ctas > 0 ? ctas : 4 * sm_count();
  moe_dispatch_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, x_stride, k, n_assign, dst_rank, dst_row, scale, b, H, s, done_slot,
      block_counter);
  return (int)cudaGetLastError();
}

extern "C" int tpb_moe_combine(size_t buf_off, const int* dst_rank, const int* dst_row,
                               const float* w, int k, int tokens, int H, void* out,
                               long long out_stride, const void* g, long long g_stride, float* dots,
                               size_t pad_off, int ready_slot, uint32_t epoch, int ctas,
                               double wait_s, uint32_t* status, void* stream) {
  TPB_NVTX("tpb_moe_combine");
  const SymmView* sv = symm_view();
  if (!sv || H % 8) return -2;
  MoePeerBufs b;
  memset(&b, 0, sizeof(b));
  for (int r = 0; r < sv->world; ++r) b.p[r] = sv->peer[r] + buf_off;
  MoeSync s = make_moe_sync(sv, pad_off, epoch, status, wait_s);
  int grid = ctas > 0 ? ctas : 4 * sm_count();
  auto kern = k <= 1 ? moe_combine_kernel<1> : k <= 2 ? moe_combine_kernel<2> : k <= 4 ? moe_combine_kernel<4>
                                                                                     : moe_combine_kernel<8>;
  kern<<<grid, 256, 0, (cudaStream_t)stream>>>(
      b, dst_rank, dst_row, w, k, tokens, H, (__nv_bfloat16*)out, out_stride,
      (const __nv_bfloat16*)g, g_stride, dots, s, ready_slot);
  return (int)cudaGetLastError();
}

extern "C" int tpb_moe_signal(size_t pad_off, int slot, uint32_t epoch, void* stream) {
  TPB_NVTX("tpb_moe_signal");
  const SymmView* sv = symm_view();
  if (!sv) return -2;
  MoeSync s = make_moe_sync(sv, pad_off, epoch, nullptr, 0);
  moe_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, slot);
  return (int)cudaGetLastError();
}

// out [cap_rows, 8] bf16 <- per-row dot products of a and b ([cap_rows, H] bf16), rows limited by *rows_dev.
extern "C" int tpb_moe_rowdot(const void* a, const void* b, void* out, const int* rows_dev, int cap_rows, int H,
                              void* stream) {
  TPB_NVTX("tpb_moe_rowdot");
  if (H % 8 || cap_rows <= 0) return -2;
  int blocks = (cap_rows + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  moe_rowdot_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                              (__nv_bfloat16*)out, rows_dev, cap_rows, H);
  return (int)cudaGetLastError();
}
