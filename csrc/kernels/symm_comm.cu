// Symmetric (peer-mapped) memory and the collectives built on it, for one process per GPU on an
// NVLink / NVSwitch box.
//
//  * Arena: every rank cudaMalloc's one arena and exports it with CUDA IPC; ranks open each
//    other's arenas, so a buffer at offset X of the local arena is reachable on rank r at
//    peer_base[r] + X. Allocation is a bump pointer that all ranks advance identically.
//  * Signal pads: a block of 32-bit flags inside the arena. A rank publishes progress by writing
//    (st.release.sys) into the pads of its peers; waiting is always a bounded poll of LOCAL memory.
//  * Kernels: all-gather by peer pulls, reduce-scatter fused with scale + AdamW + bf16 parameter
//    emit (the FSDP gradient path), all-reduce fused the same way plus parameter broadcast (the
//    DDP path), and a barrier.
//
// The reference has no peer-memory path at all: tensorplay/distributed/_symmetric_memory is a
// facade over NCCL collectives (__init__.py:228-432) and the NCCL wrapper is
// p10/src/backend/cuda/NCCLContext.cpp:231-458.
#include "sm100.cuh"
#include "tpb_api.h"

#include <string.h>

namespace tpb {

constexpr int kMaxRanks = 16;

struct SymmState {
  int world = 0, rank = 0;
  char* base = nullptr;           // local arena
  char* peer[kMaxRanks] = {};     // mapped arenas (peer[rank] == base)
  char* mc_base = nullptr;        // multicast mapping of all arenas (virtual-memory allocator only), or null
  size_t bytes = 0, used = 0;
  bool opened = false;
  bool vmm = false;               // arenas come from symm_vmm.cu (cuMemCreate), not cudaMalloc + IPC
};
static SymmState g_symm;

// Called by the virtual-memory allocator (symm_vmm.cu) once all arenas are mapped; world == 0 clears.
void symm_adopt(int world, int rank, char* const* peers, size_t bytes, char* mc_base) {
  g_symm = SymmState();
  if (world <= 0) return;
  g_symm.world = world;
  g_symm.rank = rank;
  for (int r = 0; r < world; ++r) g_symm.peer[r] = peers[r];
  g_symm.base = peers[rank];
  g_symm.bytes = bytes;
  g_symm.mc_base = mc_base;
  g_symm.opened = true;
  g_symm.vmm = true;
}
void symm_set_mc_base(char* mc_base) { g_symm.mc_base = mc_base; }

const SymmView* symm_view() {
  static SymmView v;
  if (!g_symm.base) return nullptr;
  v.world = g_symm.world;
  v.rank = g_symm.rank;
  for (int r = 0; r < kMaxRanks; ++r) v.peer[r] = g_symm.peer[r];
  return &v;
}

struct PeerPtrs {
  const char* p[kMaxRanks];
};

// ---------------------------------------------------------------- device helpers
__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Loads 8 bf16 from the same address of every rank's arena and returns their sum (added inside the
// switch with fp32 accumulation, rounded once to bf16): `p` is a multicast address.
__device__ __forceinline__ uint4 mc_ld_reduce_bf16x8(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// Stores 16 bytes to the same address of every rank's arena (`p` is a multicast address).
__device__ __forceinline__ void mc_st_v4(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Cross-rank rendezvous at kernel start. Thread 0 of block 0 publishes `epoch` into slot
// [slot_base + my_rank] of every peer's pad; every block then waits (bounded) until all local
// slots reached `epoch`. Returns false if the wait ran out of time.
struct SyncArgs {
  uint32_t* pad_local;         // local pad (flags written by peers)
  uint32_t* pad_peer[kMaxRanks];  // the same pad on every rank
  int world, rank;
  uint32_t epoch;
  unsigned long long wait_ns;
  uint32_t* status;
};

__device__ __forceinline__ bool rendezvous(const SyncArgs& s, int slot_base, uint32_t where) {
  if (blockIdx.x == 0 && threadIdx.x < s.world) {
    __threadfence_system();
    st_release_sys(s.pad_peer[threadIdx.x] + slot_base + s.rank, s.epoch);
  }
  __shared__ int ok_sh;
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (threadIdx.x < s.world) {
    if (!flag_wait_ge(s.pad_local + slot_base + threadIdx.x, s.epoch, true, s.status, s.wait_ns, where))
      ok_sh = 0;
  }
  __syncthreads();
  return ok_sh != 0;
}

// ---------------------------------------------------------------- all-gather (pull)
// out[r * shard_bytes ...] = shard of rank r. Chunks are visited starting at rank+1 so that at
// any moment the ranks pull from different peers.
__global__ void __launch_bounds__(512)
allgather_pull_kernel(PeerPtrs shards, char* __restrict__ out, size_t shard_bytes, SyncArgs s,
                      int slot_base) {
  if (!rendezvous(s, slot_base, 20)) return;
  const size_t nvec = shard_bytes / 16;
  const size_t per_rank_blocks = gridDim.x / s.world;
  const int pr = blockIdx.x / per_rank_blocks;          // which peer (offset from own rank)
  const int r = (s.rank + 1 + pr) % s.world;
  if (pr >= s.world) return;
  const size_t bid = blockIdx.x % per_rank_blocks;
  const uint4* src = reinterpret_cast<const uint4*>(shards.p[r]);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * shard_bytes);
  // NVLink latency is microseconds: keep kUnroll independent 16-byte loads in flight per thread
  constexpr int kUnroll = 8;
  const size_t stride = per_rank_blocks * blockDim.x;
  size_t i = bid * blockDim.x + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = ld_relaxed_sys_v4(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < nvec; i += stride) dst[i] = ld_relaxed_sys_v4(src + i);
}

// ---------------------------------------------------------------- all-gather (multicast push)
// Every rank stores its shard once through the multicast mapping; the switch delivers it into the
// `out` buffer of every rank (own included) at [rank * shard_bytes, ...). The rendezvous at the
// start says "my destination buffer is free and my shard is valid"; after the last block every
// rank is told that this rank's shard has landed (done_slot), which the consumer waits for.
__global__ void __launch_bounds__(512)
allgather_mc_kernel(const char* __restrict__ shard, char* __restrict__ mc_out, size_t shard_bytes, SyncArgs s,
                    int ready_slot, int done_slot, uint32_t* block_counter) {
  if (!rendezvous(s, ready_slot, 25)) return;
  const size_t nvec = shard_bytes / 16;
  const uint4* src = reinterpret_cast<const uint4*>(shard);
  uint4* dst = reinterpret_cast<uint4*>(mc_out);
  constexpr int kUnroll = 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) mc_st_v4(dst + i + u * stride, v[u]);
  }
  for (; i < nvec; i += stride) mc_st_v4(dst + i, src[i]);
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

// ---------------------------------------------------------------- one-shot all-reduce + residual + RMSNorm
// Small row-parallel outputs (decode: [rows <= a few hundred, H]): every rank holds a partial sum of
// the same [rows, H] bf16 matrix in its arena. One CTA per row: after the cross-rank rendezvous ("my
// partial is complete") each thread loads 8 elements of the SUM (one multimem.ld_reduce through the
// switch, or one load per peer), adds the residual stream, writes the new residual and, from the
// row's sum of squares, the RMS-normalised row for the next projection. All-reduce, residual add and
// norm are one launch, and every rank ends with the full result (no second phase). The partial buffers
// alternate between two arena slices from call to call, so a rank that runs ahead writes its next
// partial into the slice that no peer can still be reading; no closing rendezvous is needed.
// The epoch lives in device memory and is advanced by the kernel: the launch can be replayed from a
// CUDA graph.
struct ArNormArgs {
  const char* mc_partial;       // multicast address of the partial slice (null: plain peer loads)
  PeerPtrs peer_partial;        // the slice on every rank
  __nv_bfloat16* x;             // [rows, H] residual stream, updated in place (local, replicated)
  const __nv_bfloat16* norm_w;  // [H] or null (no norm output)
  __nv_bfloat16* h_out;         // [rows, H] normalised rows, or null
  int rows, H;
  float eps;
  uint32_t* epoch_dev;          // device word: calls completed so far
  uint32_t* block_counter;
  int slot;
};

__global__ void __launch_bounds__(1024)
allreduce_residual_norm_kernel(ArNormArgs a, SyncArgs s) {
  __shared__ int ok_sh;
  __shared__ float red[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_dev) + 1u;
  if (blockIdx.x == 0 && threadIdx.x < s.world) {
    __threadfence_system();
    st_release_sys(s.pad_peer[threadIdx.x] + a.slot + s.rank, epoch);
  }
  if (threadIdx.x == 0) ok_sh = 1;
  __syncthreads();
  if (threadIdx.x < s.world) {
    if (!flag_wait_ge(s.pad_local + a.slot + threadIdx.x, epoch, true, s.status, s.wait_ns, 28)) ok_sh = 0;
  }
  __syncthreads();
  if (ok_sh) {
    const int row = blockIdx.x;
    const int nvec = a.H / 8;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const size_t off = ((size_t)row * a.H + (size_t)v * 8) * 2;
      float f[8];
      if (a.mc_partial) {
        const uint4 u = mc_ld_reduce_bf16x8(a.mc_partial + off);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(hb[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = 0.f;
        for (int r = 0; r < s.world; ++r) {
          const uint4 u = ld_relaxed_sys_v4(a.peer_partial.p[r] + off);
          const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 t = __bfloat1622float2(hb[j]); f[2 * j] += t.x; f[2 * j + 1] += t.y; }
        }
      }
      uint4 xr = reinterpret_cast<const uint4*>(a.x + (size_t)row * a.H)[v];
      __nv_bfloat162* xb = reinterpret_cast<__nv_bfloat162*>(&xr);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(xb[j]);
        xb[j] = __floats2bfloat162_rn(t.x + f[2 * j], t.y + f[2 * j + 1]);
        const float2 q = __bfloat1622float2(xb[j]);   // the norm sees the stored (rounded) residual
        f[2 * j] = q.x; f[2 * j + 1] = q.y;
        ss += q.x * q.x + q.y * q.y;
      }
      reinterpret_cast<uint4*>(a.x + (size_t)row * a.H)[v] = xr;
    }
    if (a.h_out) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
      const float rstd = rsqrtf(tot / (float)a.H + a.eps);
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        const uint4 xr = reinterpret_cast<const uint4*>(a.x + (size_t)row * a.H)[v];
        const uint4 wr = reinterpret_cast<const uint4*>(a.norm_w)[v];
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xr);
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wr);
        uint4 o4;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = __bfloat1622float2(xb[j]), w2 = __bfloat1622float2(wb[j]);
          // same arithmetic as the stand-alone norm: x * rstd * w in fp32, rounded once
          ob[j] = __floats2bfloat162_rn(t.x * rstd * w2.x, t.y * rstd * w2.y);
        }
        reinterpret_cast<uint4*>(a.h_out + (size_t)row * a.H)[v] = o4;
      }
    }
  }
  // the last block advances the epoch for the next call
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned prev = atomicAdd(a.block_counter, 1u);
    if (prev == gridDim.x - 1) {
      *a.block_counter = 0;
      *a.epoch_dev = epoch;
    }
  }
}

// ---------------------------------------------------------------- all-to-all(v) (pull)
// Rank s keeps, in its arena, a send buffer and a table meta[d] = {byte offset in the send buffer,
// byte count} of what it has for rank d. The receiver pulls its segment from every source into `out`,
// packed in source order (offset of source s = sum of the counts of sources < s), and records the counts
// in out_bytes[world] (device memory, optional). Counts and offsets must be multiples of 16 bytes; a
// table entry that is not, or a total above out_capacity, sets the status word and moves nothing.
// After its last block a rank tells every source "I have read your buffer" (done_slot), which the
// source waits for before it rewrites its send buffer.
struct A2AMeta {
  const long long* p[kMaxRanks];  // every rank's table
};

__global__ void __launch_bounds__(512)
all_to_all_pull_kernel(PeerPtrs send, A2AMeta meta, char* __restrict__ out, size_t out_capacity,
                       long long* __restrict__ out_bytes, SyncArgs s, int ready_slot, int done_slot,
                       uint32_t* block_counter) {
  if (!rendezvous(s, ready_slot, 26)) return;
  __shared__ long long off_sh[kMaxRanks], cnt_sh[kMaxRanks], dst_sh[kMaxRanks + 1];
  __shared__ int bad_sh;
  if (threadIdx.x == 0) {
    int bad = 0;
    long long acc = 0;
    for (int r = 0; r < s.world; ++r) {
      const long long* t = meta.p[r] + 2 * s.rank;
      const long long o = *reinterpret_cast<const volatile long long*>(t);
      const long long c = *reinterpret_cast<const volatile long long*>(t + 1);
      if (o < 0 || c < 0 || (o & 15) || (c & 15)) bad = 1;
      off_sh[r] = o; cnt_sh[r] = c; dst_sh[r] = acc;
      acc += c;
    }
    dst_sh[s.world] = acc;
    if ((unsigned long long)acc > out_capacity) bad = 1;
    bad_sh = bad;
    if (bad && s.status) atomicCAS(s.status, 0u, kStatusBadArgs | (27u << 8));
    if (!bad && out_bytes && blockIdx.x == 0)
      for (int r = 0; r < s.world; ++r) out_bytes[r] = cnt_sh[r];
  }
  __syncthreads();
  if (!bad_sh) {
    const int per_rank_blocks = gridDim.x / s.world;
    const int pr = blockIdx.x / per_rank_blocks;
    if (pr < s.world) {
      const int r = (s.rank + pr) % s.world;  // own segment first: it needs no link
      const int bid = blockIdx.x % per_rank_blocks;
      const uint4* src = reinterpret_cast<const uint4*>(send.p[r] + off_sh[r]);
      uint4* dst = reinterpret_cast<uint4*>(out + dst_sh[r]);
      const size_t nvec = (size_t)cnt_sh[r] / 16;
      constexpr int kUnroll = 8;
      const size_t stride = (size_t)per_rank_blocks * blockDim.x;
      size_t i = (size_t)bid * blockDim.x + threadIdx.x;
      for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = ld_relaxed_sys_v4(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) dst[i + u * stride] = v[u];
      }
      for (; i < nvec; i += stride) dst[i] = ld_relaxed_sys_v4(src + i);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(block_counter, 1u);
    if (prev == gridDim.x - 1) {
      *block_counter = 0;
      __threadfence_system();
      for (int r = 0; r < s.world; ++r) st_release_sys(s.pad_peer[r] + done_slot + s.rank, s.epoch);
    }
  }
}

// ---------------------------------------------------------------- reduce-scatter + AdamW
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
};

__device__ __forceinline__ void adamw_elem(float& p, float& m, float& v, float g, const AdamArgs& h) {
  p *= (1.f - h.lr * h.weight_decay);
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  float denom = sqrtf(v) / sqrtf(h.bias_c2) + h.eps;
  p -= (h.lr / h.bias_c1) * (m / denom);
}

// grads.p[r] points at rank r's full bf16 gradient buffer (same offset in every arena). This
// rank owns elements [lo, lo + n) of it: it sums the N copies in fp32 in rank order, scales,
// and either applies AdamW (mode 0) writing fp32 master / moments and the bf16 parameter shard
// (+ optionally the same bf16 values into every peer's full parameter buffer: the all-reduce /
// DDP form), or (mode 1) stores the reduced fp32 gradient and its sum of squares.
// done_slot: after all blocks finished reading, the peers are told (slot done_slot + rank).
__global__ void __launch_bounds__(512)
rs_adamw_kernel(PeerPtrs grads, size_t lo, size_t n, float* __restrict__ master,
                float* __restrict__ m, float* __restrict__ v, __nv_bfloat16* __restrict__ shard_out,
                PeerPtrs bcast_out, size_t bcast_off, int do_bcast, float* __restrict__ red_out,
                float* __restrict__ sumsq, int mode, AdamArgs h, const float* clip_coef, SyncArgs s,
                int ready_slot, int done_slot, uint32_t* block_counter, int local_only,
                const char* __restrict__ mc_grads, char* __restrict__ mc_bcast) {
  // local_only: every gradient copy already sits in this GPU's memory (the copy engines pulled the
  // peers' slices and the hand-shakes ran as separate one-CTA kernels): no flags are touched here
  if (!local_only && !rendezvous(s, ready_slot, 21)) return;
  // A hand-shake kernel earlier in this stream ran out of time (status word set): the staged
  // gradient copies are then incomplete, so master weights and moments must stay untouched.
  if (local_only && s.status && *reinterpret_cast<volatile uint32_t*>(s.status) != 0u) return;
  const float gs = h.grad_scale * (clip_coef ? *clip_coef : 1.f);
  const size_t nvec = n / 8;
  float local_sq = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (mc_grads) {
      // one load, reduced over all ranks inside the switch: this rank receives its slice once instead
      // of once per peer
      const uint4 raw = mc_ld_reduce_bf16x8(reinterpret_cast<const uint4*>(mc_grads) + lo / 8 + i);
      const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(hb[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    // loads of up to eight ranks are issued together, then summed in rank order (deterministic)
    for (int r0 = 0; !mc_grads && r0 < s.world; r0 += 8) {
      uint4 raw[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int r = r0 + u;
        if (r < s.world) {
          const uint4* src = reinterpret_cast<const uint4*>(grads.p[r]) + lo / 8 + i;
          raw[u] = (r == s.rank) ? *src : ld_relaxed_sys_v4(src);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (r0 + u < s.world) {
          const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(hb[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= gs;
    if (mode == 2) {
      // plain all-reduce: the averaged bf16 slice goes into every rank's buffer at bcast_off
      uint4 o2;
      __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
      for (int j = 0; j < 4; ++j) ob2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      if (mc_bcast) {
        mc_st_v4(reinterpret_cast<uint4*>(mc_bcast + bcast_off) + lo / 8 + i, o2);  // one store reaches every rank
        continue;
      }
      for (int r = 0; r < s.world; ++r) {
        int rr = (s.rank + r) % s.world;
        uint4* dst = reinterpret_cast<uint4*>(const_cast<char*>(bcast_out.p[rr]) + bcast_off) + lo / 8 + i;
        *dst = o2;
      }
      continue;
    }
    if (mode == 1) {
      float4* ro = reinterpret_cast<float4*>(red_out) + 2 * i;
      ro[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      ro[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
      for (int j = 0; j < 8; ++j) local_sq += acc[j] * acc[j];
      continue;
    }
    float4* mp = reinterpret_cast<float4*>(master) + 2 * i;
    float4* mm = reinterpret_cast<float4*>(m) + 2 * i;
    float4* vv = reinterpret_cast<float4*>(v) + 2 * i;
    float pw[8], mw[8], vw[8];
    *reinterpret_cast<float4*>(pw) = mp[0];
    *reinterpret_cast<float4*>(pw + 4) = mp[1];
    *reinterpret_cast<float4*>(mw) = mm[0];
    *reinterpret_cast<float4*>(mw + 4) = mm[1];
    *reinterpret_cast<float4*>(vw) = vv[0];
    *reinterpret_cast<float4*>(vw + 4) = vv[1];
#pragma unroll
    for (int j = 0; j < 8; ++j) adamw_elem(pw[j], mw[j], vw[j], acc[j], h);
    mp[0] = *reinterpret_cast<float4*>(pw);
    mp[1] = *reinterpret_cast<float4*>(pw + 4);
    mm[0] = *reinterpret_cast<float4*>(mw);
    mm[1] = *reinterpret_cast<float4*>(mw + 4);
    vv[0] = *reinterpret_cast<float4*>(vw);
    vv[1] = *reinterpret_cast<float4*>(vw + 4);
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(pw[2 * j], pw[2 * j + 1]);
    if (shard_out) reinterpret_cast<uint4*>(shard_out)[i] = o;
    if (do_bcast && mc_bcast) {
      mc_st_v4(reinterpret_cast<uint4*>(mc_bcast + bcast_off) + lo / 8 + i, o);
    } else if (do_bcast) {
      for (int r = 0; r < s.world; ++r) {
        int rr = (s.rank + r) % s.world;
        uint4* dst = reinterpret_cast<uint4*>(const_cast<char*>(bcast_out.p[rr]) + bcast_off) + lo / 8 + i;
        *dst = o;
      }
    }
  }
  if (mode == 1 && sumsq) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xffffffffu, local_sq, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(sumsq, local_sq);
  }
  if (local_only) return;
  // tell the peers that this rank no longer reads their gradient buffers (and, for the
  // broadcast form, that its slice of their parameters has landed)
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

// Bounded wait until all `world` slots starting at slot_base reached `epoch` (local pad).
__global__ void wait_slots_kernel(SyncArgs s, int slot_base, uint32_t where) {
  if (threadIdx.x < s.world)
    flag_wait_ge(s.pad_local + slot_base + threadIdx.x, s.epoch, true, s.status, s.wait_ns, where);
}

// Same wait with the target read from a device word (graph-replayable callers).
__global__ void wait_slots_dev_kernel(SyncArgs s, int slot_base, const uint32_t* epoch_dev, uint32_t where) {
  if (threadIdx.x < s.world)
    flag_wait_ge(s.pad_local + slot_base + threadIdx.x, *epoch_dev, true, s.status, s.wait_ns, where);
}
__global__ void bump_kernel(uint32_t* ctr) { *ctr += 1u; }

__global__ void barrier_kernel(SyncArgs s, int slot_base) { rendezvous(s, slot_base, 22); }

// One-way signal: slot (slot_base + rank) on every rank's pad <- epoch (everything this stream did
// before, copies by the copy engines included, is complete and visible).
__global__ void signal_kernel(SyncArgs s, int slot_base) {
  if (threadIdx.x < s.world) {
    __threadfence_system();
    st_release_sys(s.pad_peer[threadIdx.x] + slot_base + s.rank, s.epoch);
  }
}

// Generic peer copy: dst (local) <- src on rank r (no rendezvous; caller orders it).
__global__ void __launch_bounds__(512)
peer_copy_kernel(const char* __restrict__ src, char* __restrict__ dst, size_t bytes) {
  const size_t nvec = bytes / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x)
    reinterpret_cast<uint4*>(dst)[i] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(src) + i);
}

static SyncArgs make_sync(size_t pad_off, uint32_t epoch, uint32_t* status, double wait_s) {
  SyncArgs s;
  memset(&s, 0, sizeof(s));
  s.world = g_symm.world;
  s.rank = g_symm.rank;
  s.pad_local = reinterpret_cast<uint32_t*>(g_symm.base + pad_off);
  for (int r = 0; r < g_symm.world; ++r)
    s.pad_peer[r] = reinterpret_cast<uint32_t*>(g_symm.peer[r] + pad_off);
  s.epoch = epoch;
  s.wait_ns = wait_s > 0 ? (unsigned long long)(wait_s * 1e9) : kDefaultWaitNs;
  s.status = status;
  return s;
}

}  // namespace tpb

using namespace tpb;

// ------------------------------------------------------------------ arena management (host)
// Returns 0 and fills handle_out (64 bytes) with the IPC handle of the new arena.
extern "C" int tpb_symm_create(int world, int rank, size_t bytes, void* handle_out) {
  if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -2;
  if (g_symm.base) return -4;  // already created
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return (int)e;
  g_symm.world = world;
  g_symm.rank = rank;
  g_symm.base = static_cast<char*>(p);
  g_symm.bytes = bytes;
  g_symm.used = 0;
  g_symm.peer[rank] = g_symm.base;
  if (world > 1) {
    cudaIpcMemHandle_t h;
    e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) return (int)e;
    memcpy(handle_out, &h, sizeof(h));
  } else {
    memset(handle_out, 0, 64);
  }
  return 0;
}

// handles: world * 64 bytes, rank-major (as gathered from tpb_symm_create on every rank).
extern "C" int tpb_symm_open(const void* handles) {
  if (!g_symm.base) return -4;
  for (int r = 0; r < g_symm.world; ++r) {
    if (r == g_symm.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const char*>(handles) + 64 * r, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return (int)e;
    g_symm.peer[r] = static_cast<char*>(p);
  }
  g_symm.opened = true;
  return 0;
}

extern "C" int tpb_symm_vmm_destroy();
extern "C" int tpb_symm_destroy() {
  if (!g_symm.base) return 0;
  if (g_symm.vmm) return tpb_symm_vmm_destroy();
  for (int r = 0; r < g_symm.world; ++r)
    if (r != g_symm.rank && g_symm.peer[r]) cudaIpcCloseMemHandle(g_symm.peer[r]);
  cudaFree(g_symm.base);
  g_symm = SymmState();
  return 0;
}

// Bump allocation (256-byte aligned). Returns the offset, or (size_t)-1 when the arena is full.
extern "C" size_t tpb_symm_alloc(size_t bytes) {
  size_t off = (g_symm.used + 255) & ~size_t(255);
  if (!g_symm.base || off + bytes > g_symm.bytes) return (size_t)-1;
  g_symm.used = off + bytes;
  return off;
}
extern "C" void* tpb_symm_ptr(int rank, size_t off) {
  if (!g_symm.base || rank < 0 || rank >= g_symm.world) return nullptr;
  return g_symm.peer[rank] + off;
}
extern "C" size_t tpb_symm_used() { return g_symm.used; }

// ------------------------------------------------------------------ collectives
// Multicast (in-switch) forms of the kernels are used when the arena has a multicast mapping and
// they are not switched off (tpb_symm_set_multicast(0): plain peer loads and stores, the form that
// tests of rank failure must use).
static bool g_mc_enabled = true;
static bool use_mc() { return g_mc_enabled && g_symm.mc_base != nullptr && g_symm.world > 1; }
extern "C" int tpb_symm_set_multicast(int on) {
  g_mc_enabled = on != 0;
  return 0;
}
extern "C" int tpb_symm_has_multicast() { return g_symm.mc_base != nullptr && g_symm.world > 1; }
extern "C" void* tpb_symm_mc_ptr(size_t off) { return g_symm.mc_base ? g_symm.mc_base + off : nullptr; }

static PeerPtrs peers_at(size_t off) {
  PeerPtrs pp;
  memset(&pp, 0, sizeof(pp));
  for (int r = 0; r < g_symm.world; ++r) pp.p[r] = g_symm.peer[r] + off;
  return pp;
}

// out (any local device pointer) <- concatenation over ranks of the shard at arena offset
// shard_off. pad_off/slot_base: `world` consecutive flag slots used as the "shards are valid
// at epoch" rendezvous.
extern "C" int tpb_symm_allgather(size_t shard_off, size_t shard_bytes, void* out, size_t pad_off,
                                  int slot_base, uint32_t epoch, int ctas, double wait_s,
                                  uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_allgather");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  if (shard_bytes % 16 || (reinterpret_cast<uintptr_t>(out) & 15)) return -2;
  int per_rank = ctas > 0 ? ctas : 8;
  int grid = per_rank * g_symm.world;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  allgather_pull_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(
      peers_at(shard_off), static_cast<char*>(out), shard_bytes, s, slot_base);
  return (int)cudaGetLastError();
}

// All-gather by multicast stores (arenas of the virtual-memory allocator with a multicast mapping
// only). shard: local device pointer; the result appears at arena offset out_off on every rank once
// its done_slot flags reached `epoch` (wait with tpb_symm_wait_slots). ready_slot / done_slot:
// `world` flag slots each.
extern "C" int tpb_symm_allgather_mc(const void* shard, size_t shard_bytes, size_t out_off, size_t pad_off,
                                     int ready_slot, int done_slot, uint32_t epoch, uint32_t* block_counter,
                                     int ctas, double wait_s, uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_allgather_mc");
  if (!g_symm.mc_base || g_symm.world < 2) return -4;
  if (shard_bytes % 16 || (reinterpret_cast<uintptr_t>(shard) & 15) || out_off % 16) return -2;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  allgather_mc_kernel<<<ctas > 0 ? ctas : 32, 512, 0, (cudaStream_t)stream>>>(
      static_cast<const char*>(shard), g_symm.mc_base + out_off + (size_t)g_symm.rank * shard_bytes, shard_bytes, s,
      ready_slot, done_slot, block_counter);
  return (int)cudaGetLastError();
}

// x[rows, H] += sum over ranks of the partial at arena offset partial_off; h_out = rmsnorm(x) * norm_w
// (norm_w / h_out may be null). One CTA per row. epoch_dev: device word owned by the caller (starts at 0,
// advanced here); slot: `world` flag slots; block_counter: zeroed device word. Consecutive calls must
// alternate between two partial slices (see the kernel's comment).
extern "C" int tpb_symm_allreduce_residual_norm(size_t partial_off, void* x, const void* norm_w, void* h_out,
                                                int rows, int H, float eps, size_t pad_off, int slot,
                                                uint32_t* epoch_dev, uint32_t* block_counter, double wait_s,
                                                uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_allreduce_residual_norm");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  if (rows <= 0) return 0;
  if (H % 8 || partial_off % 16 || (h_out && !norm_w)) return -2;
  ArNormArgs a;
  memset(&a, 0, sizeof(a));
  a.mc_partial = use_mc() ? g_symm.mc_base + partial_off : nullptr;
  a.peer_partial = peers_at(partial_off);
  a.x = (__nv_bfloat16*)x; a.norm_w = (const __nv_bfloat16*)norm_w; a.h_out = (__nv_bfloat16*)h_out;
  a.rows = rows; a.H = H; a.eps = eps; a.epoch_dev = epoch_dev; a.block_counter = block_counter; a.slot = slot;
  SyncArgs s = make_sync(pad_off, 0, status, wait_s);
  int threads = H / 8;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : (threads + 31) / 32 * 32);
  allreduce_residual_norm_kernel<<<rows, threads, 0, (cudaStream_t)stream>>>(a, s);
  return (int)cudaGetLastError();
}

// All-to-all with per-pair byte counts. send_off: arena offset of the send buffer; meta_off: arena
// offset of this rank's table of `world` {offset, bytes} pairs (int64, written by the caller before the
// launch, stream-ordered). out: local pointer with room for out_capacity bytes; out_bytes: optional device
// int64[world]. ready_slot / done_slot: `world` flag slots each; wait on done_slot (tpb_symm_wait_slots)
// before rewriting the send buffer or the table.
extern "C" int tpb_symm_all_to_all(size_t send_off, size_t meta_off, void* out, size_t out_capacity,
                                   long long* out_bytes, size_t pad_off, int ready_slot, int done_slot,
                                   uint32_t epoch, uint32_t* block_counter, int ctas, double wait_s,
                                   uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_all_to_all");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || send_off % 16 || meta_off % 8) return -2;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  A2AMeta meta;
  memset(&meta, 0, sizeof(meta));
  for (int r = 0; r < g_symm.world; ++r) meta.p[r] = reinterpret_cast<const long long*>(g_symm.peer[r] + meta_off);
  const int per_rank = ctas > 0 ? ctas : 8;
  all_to_all_pull_kernel<<<per_rank * g_symm.world, 512, 0, (cudaStream_t)stream>>>(
      peers_at(send_off), meta, static_cast<char*>(out), out_capacity, out_bytes, s, ready_slot, done_slot,
      block_counter);
  return (int)cudaGetLastError();
}

// Fused reduce-scatter + AdamW over the bf16 gradient buffer at arena offset grad_off.
//   mode 0: update master/m/v (local fp32 pointers, n elements), write bf16 shard to shard_out
//           (local pointer, may be null); if bcast_off != (size_t)-1 also write the bf16 values
//           into every rank's buffer at arena offset bcast_off (+ lo): all-reduce/DDP form.
//   mode 1: write the reduced, scaled fp32 gradient to red_out and add its squares to sumsq.
//   mode 2: all-reduce: write the reduced, scaled bf16 values into every rank's buffer at
//           arena offset bcast_off (may equal grad_off: in place).
// ready_slot / done_slot: `world` flag slots each.
extern "C" int tpb_symm_rs_adamw(size_t grad_off, size_t lo, size_t n, float* master, float* m,
                                 float* v, void* shard_out, size_t bcast_off, float* red_out,
                                 float* sumsq, int mode, float lr, float beta1, float beta2,
                                 float eps, float wd, int step, float grad_scale,
                                 const float* clip_coef, size_t pad_off, int ready_slot,
                                 int done_slot, uint32_t epoch, uint32_t* block_counter, int ctas,
                                 double wait_s, uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_rs_adamw");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  if (n % 8 || lo % 8) return -2;
  AdamArgs h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = wd;
  h.bias_c1 = 1.f - powf(beta1, (float)step);
  h.bias_c2 = 1.f - powf(beta2, (float)step);
  h.grad_scale = grad_scale;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  int grid = ctas > 0 ? ctas : 64;
  int do_bcast = bcast_off != (size_t)-1;
  rs_adamw_kernel<<<grid, 512, 0, (cudaStream_t)stream>>>(
      peers_at(grad_off), lo, n, master, m, v, (__nv_bfloat16*)shard_out,
      do_bcast ? peers_at(0) : peers_at(0), do_bcast ? bcast_off : 0, do_bcast, red_out, sumsq, mode,
      h, clip_coef, s, ready_slot, done_slot, block_counter, 0,
      use_mc() ? g_symm.mc_base + grad_off : nullptr, use_mc() ? g_symm.mc_base : nullptr);
  return (int)cudaGetLastError();
}

extern "C" int tpb_symm_wait_slots(size_t pad_off, int slot_base, uint32_t epoch, double wait_s,
                                   uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_wait_slots");
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  wait_slots_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, slot_base, 23);
  return (int)cudaGetLastError();
}

// Wait until all `world` slots reached the value stored at epoch_dev (device memory).
extern "C" int tpb_symm_wait_slots_dev(size_t pad_off, int slot_base, const uint32_t* epoch_dev, double wait_s,
                                       uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_wait_slots_dev");
  SyncArgs s = make_sync(pad_off, 0, status, wait_s);
  wait_slots_dev_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, slot_base, epoch_dev, 24);
  return (int)cudaGetLastError();
}
// *ctr += 1 in stream order (advances a device-side epoch after the launch that used it).
extern "C" int tpb_symm_bump(uint32_t* ctr, void* stream) {
  TPB_NVTX("tpb_symm_bump");
  bump_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(ctr);
  return (int)cudaGetLastError();
}

extern "C" int tpb_symm_barrier(size_t pad_off, int slot_base, uint32_t epoch, double wait_s,
                                uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_barrier");
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(s, slot_base);
  return (int)cudaGetLastError();
}

// dst (local) <- [src_off, src_off + bytes) of rank src_rank's arena.
extern "C" int tpb_symm_peer_copy(int src_rank, size_t src_off, void* dst, size_t bytes, int ctas,
                                  void* stream) {
  TPB_NVTX("tpb_symm_peer_copy");
  if (bytes % 16) return -2;
  peer_copy_kernel<<<ctas > 0 ? ctas : 32, 512, 0, (cudaStream_t)stream>>>(
      g_symm.peer[src_rank] + src_off, static_cast<char*>(dst), bytes);
  return (int)cudaGetLastError();
}

// Overlap mode of the reduce + AdamW kernel (both transports): `threads` per CTA (256 leaves room
// beside a persistent GEMM CTA in the register file) and whether it accepts the GEMM's shared-memory
// carveout, i.e. may share an SM with it instead of waiting for the GEMM's CTAs to leave.
static int g_rs_threads = 512;
static bool g_rs_cfg_dirty = false;
static bool g_rs_max_shared = false;
extern "C" int tpb_symm_set_overlap(int threads, int max_shared) {
  if (threads != 128 && threads != 256 && threads != 512) return -1;
  g_rs_threads = threads;
  g_rs_max_shared = max_shared != 0;
  g_rs_cfg_dirty = true;
  return 0;
}
static int rs_threads() {
  if (g_rs_cfg_dirty) {
    cudaFuncSetAttribute(rs_adamw_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         g_rs_max_shared ? (int)cudaSharedmemCarveoutMaxShared : (int)cudaSharedmemCarveoutDefault);
    g_rs_cfg_dirty = false;
  }
  return g_rs_threads;
}

// ---------------------------------------------------------------- copy-engine variants
// Bulk transfers by the GPU's copy engines instead of SM kernels: the NVLink traffic then costs no
// SM time and never competes with the persistent GEMMs for their SMs. The hand-shakes stay on the
// device (one-CTA kernels in the same stream); the arithmetic stays fused in one kernel that reads
// only local memory.

// All-gather: out[r * shard_bytes ...] = shard of rank r (peers are visited starting at rank + 1).
extern "C" int tpb_symm_allgather_ce(size_t shard_off, size_t shard_bytes, void* out, size_t pad_off,
                                     int slot_base, uint32_t epoch, double wait_s, uint32_t* status,
                                     void* stream) {
  TPB_NVTX("tpb_symm_allgather_ce");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  cudaStream_t st = (cudaStream_t)stream;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  barrier_kernel<<<1, 32, 0, st>>>(s, slot_base);  // every rank's shard is valid at this epoch
  for (int k = 1; k <= g_symm.world; ++k) {
    const int r = (g_symm.rank + k) % g_symm.world;
    cudaError_t e = cudaMemcpyAsync(static_cast<char*>(out) + (size_t)r * shard_bytes,
                                    g_symm.peer[r] + shard_off, shard_bytes, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaGetLastError();
}

// Reduce-scatter + AdamW: the peers' slices [lo, lo + n) of the bf16 gradient buffer at grad_off are
// pulled into `staging` ([world][n] bf16, local), the peers are told that their buffers are free, and
// the fused reduce + scale + AdamW kernel runs on local memory only. Modes as in tpb_symm_rs_adamw
// (0 and 1; the broadcast forms need peer stores and stay with the SM kernel).
extern "C" int tpb_symm_rs_adamw_ce(size_t grad_off, size_t lo, size_t n, void* staging, float* master,
                                    float* m, float* v, void* shard_out, float* red_out, float* sumsq,
                                    int mode, float lr, float beta1, float beta2, float eps, float wd,
                                    int step, float grad_scale, const float* clip_coef, size_t pad_off,
                                    int ready_slot, int done_slot, uint32_t epoch, int ctas,
                                    double wait_s, uint32_t* status, void* stream) {
  TPB_NVTX("tpb_symm_rs_adamw_ce");
  if (!g_symm.opened && g_symm.world > 1) return -4;
  if (n % 8 || lo % 8 || (mode != 0 && mode != 1)) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  SyncArgs s = make_sync(pad_off, epoch, status, wait_s);
  barrier_kernel<<<1, 32, 0, st>>>(s, ready_slot);  // every rank's gradients are complete
  PeerPtrs local;
  memset(&local, 0, sizeof(local));
  for (int k = 0; k < g_symm.world; ++k) {
    const int r = (g_symm.rank + k) % g_symm.world;
    if (r == g_symm.rank) {
      local.p[r] = g_symm.base + grad_off;  // own copy is read in place
      continue;
    }
    char* dst = static_cast<char*>(staging) + (size_t)r * n * 2;
    cudaError_t e = cudaMemcpyAsync(dst, g_symm.peer[r] + grad_off + lo * 2, n * 2, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return (int)e;
    local.p[r] = dst - lo * 2;  // the kernel indexes every copy at element lo + i
  }
  signal_kernel<<<1, 32, 0, st>>>(s, done_slot);  // the peers' gradient buffers may be reused
  AdamArgs h;
  h.lr = lr; h.beta1 = beta1; h.beta2 = beta2; h.eps = eps; h.weight_decay = wd;
  h.bias_c1 = 1.f - powf(beta1, (float)step);
  h.bias_c2 = 1.f - powf(beta2, (float)step);
  h.grad_scale = grad_scale;
  const int grid = ctas > 0 ? ctas : 148;
  rs_adamw_kernel<<<grid, rs_threads(), 0, st>>>(local, lo, n, master, m, v, (__nv_bfloat16*)shard_out, local, 0, 0,
                                        red_out, sumsq, mode, h, clip_coef, s, ready_slot, done_slot,
                                        nullptr, 1, nullptr, nullptr);
  return (int)cudaGetLastError();
}
