// Context-parallel (ring) attention support: merge of two attention partials by their
// log-sum-exp. Each ring step attends the local queries to one rank's K/V chunk (pulled from
// peer memory) and folds the partial output into an fp32 accumulator with this kernel.
//
// Capability reference: tensorplay/distributed/tensor/experimental/_context_parallel/
// _attention.py:98-170 (_partial_update / _SDPAMerger).
#include <math_constants.h>

#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {
namespace {

// One warp per (b, t, h): acc = acc * w_old + part * w_new, lse_acc = logaddexp(lse_acc, lse_part).
// first != 0 initialises the accumulator from the partial.
__global__ void __launch_bounds__(256)
attn_merge_kernel(float* __restrict__ acc, float* __restrict__ lse_acc,
                  const __nv_bfloat16* __restrict__ part, const float* __restrict__ lse_part,
                  int B, int T, int H, int D, long long p_tok, long long p_head, long long p_batch,
                  int lse_acc_stride, int lse_part_stride, int first) {
  const long long w = ((long long)blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)B * T * H) return;
  const int h = (int)(w % H);
  const long long bt = w / H;
  const int t = (int)(bt % T);
  const int b = (int)(bt / T);
  float* a = acc + ((long long)(b * (long long)T + t) * H + h) * D;
  const __nv_bfloat16* pr = part + b * p_batch + t * p_tok + h * p_head;
  const long long la = ((long long)b * H + h) * lse_acc_stride + t;
  const float ln = lse_part[((long long)b * H + h) * lse_part_stride + t];
  float w_old = 0.f, w_new = 1.f, lse = ln;
  if (!first) {
    const float lo = lse_acc[la];
    const float mx = fmaxf(lo, ln);
    if (mx == -CUDART_INF_F) {
      w_old = 0.f; w_new = 0.f; lse = -CUDART_INF_F;
    } else {
      const float eo = __expf(lo - mx), en = __expf(ln - mx);
      const float s = eo + en;
      w_old = eo / s; w_new = en / s;
      lse = mx + __logf(s);
    }
  } else if (ln == -CUDART_INF_F) {
    w_new = 0.f;
  }
  for (int d = lane * 2; d < D; d += 64) {
    const float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pr + d));
    float2 av = first ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(a + d);
    av.x = av.x * w_old + pv.x * w_new;
    av.y = av.y * w_old + pv.y * w_new;
    *reinterpret_cast<float2*>(a + d) = av;
  }
  if (lane == 0) lse_acc[la] = lse;
}

}  // namespace
}  // namespace tpb

// acc: fp32 [B, T, H, D] contiguous; lse_acc: fp32 [B, H, lse_acc_stride]; part: bf16 [B, T, H, D]
// by strides; lse_part: fp32 [B, H, lse_part_stride].
extern "C" int tpb_attn_merge(float* acc, float* lse_acc, const void* part, const float* lse_part,
                              int B, int T, int H, int D, long long p_tok, long long p_head,
                              long long p_batch, int lse_acc_stride, int lse_part_stride, int first,
                              void* stream) {
  TPB_NVTX("tpb_attn_merge");
  if (B <= 0 || T <= 0 || H <= 0) return 0;
  if (D <= 0 || (D & 1) || ((p_tok | p_head | p_batch) & 1)) return -1;
  const long long warps = (long long)B * T * H;
  const int grid = (int)((warps * 32 + 255) / 256);
  tpb::attn_merge_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      acc, lse_acc, static_cast<const __nv_bfloat16*>(part), lse_part, B, T, H, D, p_tok, p_head,
      p_batch, lse_acc_stride, lse_part_stride, first);
  return (int)cudaGetLastError();
}
