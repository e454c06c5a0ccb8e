// Detection kernels: non-maximum suppression and RoIAlign (forward / backward).
//
// Capability reference: tensorplay/vision/ops/boxes.py (nms, batched_nms, box_iou),
// tensorplay/vision/ops/roi_align.py and the device kernels behind them under
// p10/src/backend/cuda/vision. Plain CUDA compute (no tensor cores): NMS is a bit-matrix of pairwise
// overlaps followed by a single-CTA scan that stays on the device (no host round trip between the
// two), RoIAlign is one thread per output element with bilinear taps, its backward scatters with
// fp32 atomics.
#include "sm100.cuh"
#include "tpb_api.h"

namespace tpb {
namespace {

constexpr int kNmsTile = 64;

__device__ __forceinline__ float box_iou_dev(const float4 a, const float4 b) {
  const float l = fmaxf(a.x, b.x), t = fmaxf(a.y, b.y), r = fminf(a.z, b.z), d = fminf(a.w, b.w);
  const float w = fmaxf(r - l, 0.f), h = fmaxf(d - t, 0.f);
  const float inter = w * h;
  const float ua = (a.z - a.x) * (a.w - a.y) + (b.z - b.x) * (b.w - b.y) - inter;
  return ua > 0.f ? inter / ua : 0.f;
}

// boxes are visited in the order `order` (scores descending). mask[i][w] bit j: box order[w*64+j]
// overlaps box order[i] by more than the threshold and comes later in the order.
__global__ void __launch_bounds__(kNmsTile)
nms_mask_kernel(const float4* __restrict__ boxes, const long long* __restrict__ order, int n, float thr,
                unsigned long long* __restrict__ mask, int words) {
  const int row0 = blockIdx.y * kNmsTile, col0 = blockIdx.x * kNmsTile;
  if (col0 + kNmsTile <= row0) {  // all columns come earlier in the order: nothing to suppress
    const int i = row0 + threadIdx.x;
    if (i < n) mask[(size_t)i * words + blockIdx.x] = 0ull;
    return;
  }
  __shared__ float4 cols[kNmsTile];
  const int cn = min(kNmsTile, n - col0);
  if ((int)threadIdx.x < cn) cols[threadIdx.x] = boxes[order[col0 + threadIdx.x]];
  __syncthreads();
  const int i = row0 + threadIdx.x;
  if (i >= n) return;
  const float4 me = boxes[order[i]];
  unsigned long long bits = 0ull;
  for (int j = 0; j < cn; ++j)
    if (col0 + j > i && box_iou_dev(me, cols[j]) > thr) bits |= 1ull << j;
  mask[(size_t)i * words + blockIdx.x] = bits;
}

// One CTA walks the boxes in order; `removed` lives in shared memory. keep[i] = 1 when box order[i] survives;
// *n_keep counts them.
__global__ void __launch_bounds__(1024)
nms_scan_kernel(const unsigned long long* __restrict__ mask, int n, int words, unsigned char* __restrict__ keep,
                int* __restrict__ n_keep) {
  extern __shared__ unsigned long long removed[];
  for (int w = threadIdx.x; w < words; w += blockDim.x) removed[w] = 0ull;
  __shared__ int kept;
  if (threadIdx.x == 0) kept = 0;
  __syncthreads();
  for (int i = 0; i < n; ++i) {
    const bool alive = !((removed[i >> 6] >> (i & 63)) & 1ull);   // every thread reads the same word
    __syncthreads();                                               // ... before anyone updates it
    if (alive) {
      for (int w = (i >> 6) + threadIdx.x; w < words; w += blockDim.x) removed[w] |= mask[(size_t)i * words + w];
      if (threadIdx.x == 0) { keep[i] = 1; ++kept; }
    } else if (threadIdx.x == 0) {
      keep[i] = 0;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) *n_keep = kept;
}

// ------------------------------------------------------------------ RoIAlign
struct RoiAlignParams {
  int K, C, H, W, ph, pw, sampling_ratio, aligned;
  float spatial_scale;
};

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16(v); }

// Bilinear tap positions and weights of a sample point; false when the point lies outside the map by more
// than one pixel (it then contributes zero).
__device__ __forceinline__ bool bilinear_taps(float y, float x, int H, int W, int& y0, int& x0, int& y1, int& x1,
                                              float& w00, float& w01, float& w10, float& w11) {
  if (y < -1.f || y > (float)H || x < -1.f || x > (float)W) return false;
  y = fmaxf(y, 0.f);
  x = fmaxf(x, 0.f);
  y0 = (int)y; x0 = (int)x;
  if (y0 >= H - 1) { y0 = y1 = H - 1; y = (float)y0; } else y1 = y0 + 1;
  if (x0 >= W - 1) { x0 = x1 = W - 1; x = (float)x0; } else x1 = x0 + 1;
  const float ly = y - y0, lx = x - x0, hy = 1.f - ly, hx = 1.f - lx;
  w00 = hy * hx; w01 = hy * lx; w10 = ly * hx; w11 = ly * lx;
  return true;
}

struct RoiGeom {
  float start_w, start_h, bin_w, bin_h;
  int grid_h, grid_w, batch;
};

__device__ __forceinline__ RoiGeom roi_geom(const float* roi, const RoiAlignParams& p) {
  RoiGeom g;
  g.batch = (int)roi[0];
  const float off = p.aligned ? 0.5f : 0.f;
  g.start_w = roi[1] * p.spatial_scale - off;
  g.start_h = roi[2] * p.spatial_scale - off;
  float rw = roi[3] * p.spatial_scale - off - g.start_w;
  float rh = roi[4] * p.spatial_scale - off - g.start_h;
  if (!p.aligned) { rw = fmaxf(rw, 1.f); rh = fmaxf(rh, 1.f); }
  g.bin_h = rh / p.ph;
  g.bin_w = rw / p.pw;
  g.grid_h = p.sampling_ratio > 0 ? p.sampling_ratio : (int)ceilf(rh / p.ph);
  g.grid_w = p.sampling_ratio > 0 ? p.sampling_ratio : (int)ceilf(rw / p.pw);
  return g;
}

template <typename T>
__global__ void __launch_bounds__(256)
roi_align_fwd_kernel(const T* __restrict__ x, const float* __restrict__ rois, T* __restrict__ y, RoiAlignParams p,
                     int n_batch) {
  const long long total = (long long)p.K * p.C * p.ph * p.pw;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int pwi = (int)(i % p.pw);
    const int phi = (int)((i / p.pw) % p.ph);
    const int c = (int)((i / ((long long)p.pw * p.ph)) % p.C);
    const int k = (int)(i / ((long long)p.pw * p.ph * p.C));
    const RoiGeom g = roi_geom(rois + (size_t)k * 5, p);
    float acc = 0.f;
    if (TPB_DBG_CHECK(g.batch >= 0 && g.batch < n_batch, 45)) {
      const T* plane = x + ((size_t)g.batch * p.C + c) * p.H * p.W;
      for (int iy = 0; iy < g.grid_h; ++iy) {
        const float yy = g.start_h + phi * g.bin_h + (iy + 0.5f) * g.bin_h / g.grid_h;
        for (int ix = 0; ix < g.grid_w; ++ix) {
          const float xx = g.start_w + pwi * g.bin_w + (ix + 0.5f) * g.bin_w / g.grid_w;
          int y0, x0, y1, x1;
          float w00, w01, w10, w11;
          if (!bilinear_taps(yy, xx, p.H, p.W, y0, x0, y1, x1, w00, w01, w10, w11)) continue;
          acc += w00 * ldf(plane + y0 * p.W + x0) + w01 * ldf(plane + y0 * p.W + x1) +
                 w10 * ldf(plane + y1 * p.W + x0) + w11 * ldf(plane + y1 * p.W + x1);
        }
      }
      const int cnt = max(g.grid_h * g.grid_w, 1);
      acc /= cnt;
    }
    stf(y + i, acc);
  }
}

// dx (fp32, zero-initialised by the caller) += scatter of dy through the same taps.
template <typename T>
__global__ void __launch_bounds__(256)
roi_align_bwd_kernel(const T* __restrict__ dy, const float* __restrict__ rois, float* __restrict__ dx,
                     RoiAlignParams p, int n_batch) {
  const long long total = (long long)p.K * p.C * p.ph * p.pw;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const int pwi = (int)(i % p.pw);
    const int phi = (int)((i / p.pw) % p.ph);
    const int c = (int)((i / ((long long)p.pw * p.ph)) % p.C);
    const int k = (int)(i / ((long long)p.pw * p.ph * p.C));
    const RoiGeom g = roi_geom(rois + (size_t)k * 5, p);
    if (!TPB_DBG_CHECK(g.batch >= 0 && g.batch < n_batch, 46)) continue;
    float* plane = dx + ((size_t)g.batch * p.C + c) * p.H * p.W;
    const float gy = ldf(dy + i) / max(g.grid_h * g.grid_w, 1);
    for (int iy = 0; iy < g.grid_h; ++iy) {
      const float yy = g.start_h + phi * g.bin_h + (iy + 0.5f) * g.bin_h / g.grid_h;
      for (int ix = 0; ix < g.grid_w; ++ix) {
        const float xx = g.start_w + pwi * g.bin_w + (ix + 0.5f) * g.bin_w / g.grid_w;
        int y0, x0, y1, x1;
        float w00, w01, w10, w11;
        if (!bilinear_taps(yy, xx, p.H, p.W, y0, x0, y1, x1, w00, w01, w10, w11)) continue;
        atomicAdd(plane + y0 * p.W + x0, gy * w00);
        atomicAdd(plane + y0 * p.W + x1, gy * w01);
        atomicAdd(plane + y1 * p.W + x0, gy * w10);
        atomicAdd(plane + y1 * p.W + x1, gy * w11);
      }
    }
  }
}

}  // namespace
}  // namespace tpb

using namespace tpb;

extern "C" long long tpb_nms_workspace_bytes(int n) {
  const long long words = (n + 63) / 64;
  return (long long)n * words * 8;
}

// boxes fp32 [n, 4] (x1, y1, x2, y2); order int64 [n]: indices by descending score; mask: workspace of
// tpb_nms_workspace_bytes(n); keep uint8 [n] (in `order` positions); n_keep int32 [1].
extern "C" int tpb_nms(const float* boxes, const long long* order, int n, float iou_threshold, void* mask,
                       unsigned char* keep, int* n_keep, void* stream) {
  TPB_NVTX("tpb_nms");
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(boxes) & 15) return -2;
  const int words = (n + 63) / 64;
  if ((size_t)words * 8 > 200 * 1024) return -2;   // the scan keeps one bit per box in shared memory
  auto st = static_cast<cudaStream_t>(stream);
  dim3 grid(words, words);
  nms_mask_kernel<<<grid, kNmsTile, 0, st>>>(reinterpret_cast<const float4*>(boxes), order, n, iou_threshold,
                                             static_cast<unsigned long long*>(mask), words);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(nms_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int threads = words >= 1024 ? 1024 : (words >= 256 ? 256 : 64);
  nms_scan_kernel<<<1, threads, (size_t)words * 8, st>>>(static_cast<const unsigned long long*>(mask), n, words,
                                                         keep, n_keep);
  return (int)cudaGetLastError();
}

extern "C" int tpb_roi_align_fwd(const void* x, const float* rois, void* y, int bf16, int N, int C, int H, int W,
                                 int K, int ph, int pw, float spatial_scale, int sampling_ratio, int aligned,
                                 void* stream) {
  TPB_NVTX("tpb_roi_align_fwd");
  if (K <= 0 || C <= 0) return 0;
  if (ph <= 0 || pw <= 0 || H <= 0 || W <= 0) return -2;
  RoiAlignParams p{K, C, H, W, ph, pw, sampling_ratio, aligned, spatial_scale};
  const long long total = (long long)K * C * ph * pw;
  const int grid = (int)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
  auto st = static_cast<cudaStream_t>(stream);
  if (bf16)
    roi_align_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, rois, (__nv_bfloat16*)y, p, N);
  else
    roi_align_fwd_kernel<float><<<grid, 256, 0, st>>>((const float*)x, rois, (float*)y, p, N);
  return (int)cudaGetLastError();
}

extern "C" int tpb_roi_align_bwd(const void* dy, const float* rois, float* dx, int bf16, int N, int C, int H, int W,
                                 int K, int ph, int pw, float spatial_scale, int sampling_ratio, int aligned,
                                 void* stream) {
  TPB_NVTX("tpb_roi_align_bwd");
  if (K <= 0 || C <= 0) return 0;
  if (ph <= 0 || pw <= 0 || H <= 0 || W <= 0) return -2;
  RoiAlignParams p{K, C, H, W, ph, pw, sampling_ratio, aligned, spatial_scale};
  const long long total = (long long)K * C * ph * pw;
  const int grid = (int)((total + 255) / 256 < 148 * 32 ? (total + 255) / 256 : 148 * 32);
  auto st = static_cast<cudaStream_t>(stream);
  if (bf16)
    roi_align_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dy, rois, dx, p, N);
  else
    roi_align_bwd_kernel<float><<<grid, 256, 0, st>>>((const float*)dy, rois, dx, p, N);
  return (int)cudaGetLastError();
}
