// Allocation-free entry point (no counterpart in the reference framework).
//
// Who needs it: callers that are not allowed to create device memory at the moment they need
// the operation - a serving process that handed every free byte of the GPU to its KV-cache pool
// at start-up, a plug-in running inside a host application whose allocator it must not touch, or
// a latency-critical loop that cannot afford the implicit device synchronisation of cudaMalloc /
// cudaFree. The regular tpb_rmsnorm_bwd wants a caller-provided scratch buffer for the
// per-block partial sums of the weight gradient; this variant keeps that scratch inside the
// library instead.
//
// How: the scratch is a file-scope `static __device__` array of
// TPB_NOALLOC_RMSNORM_MAX_FLOATS floats (9.25 MiB), so every GPU that loads the library holds
// it from load time until the process exits. The entry point never calls cudaMalloc, cudaFree
// or any allocating library routine; inputs and outputs are still supplied by the caller.
//
// Set-up: the first call on each device looks up the array's device address (with that device
// current) and caches it. Make that first call outside of any stream capture.
//
// Limits and sharing:
//   * rows * H is unrestricted, but blocks * H must fit the array: H % 8 == 0, H <= 8192 and the
//     launch uses at most TPB_NOALLOC_RMSNORM_MAX_BLOCKS blocks. Larger problems are rejected
//     with TPB_NOALLOC_TOO_LARGE before anything is launched (see tpb_noalloc_strerror).
//   * All calls on a device share the one array and it keeps the previous call's contents. The
//     kernel overwrites every partial row it later reads, so nothing has to be cleared between
//     calls; but two calls that overlap on the GPU (different streams, no ordering between them)
//     race on the scratch and produce wrong weight gradients. Order such calls with events, or
//     issue them on one stream.
#pragma once
#include <stdint.h>

#define TPB_NOALLOC_RMSNORM_MAX_BLOCKS 296
#define TPB_NOALLOC_RMSNORM_MAX_H 8192
#define TPB_NOALLOC_RMSNORM_MAX_FLOATS (TPB_NOALLOC_RMSNORM_MAX_BLOCKS * TPB_NOALLOC_RMSNORM_MAX_H)

#define TPB_NOALLOC_TOO_LARGE (-22)   // H or the block count exceeds the built-in scratch
#define TPB_NOALLOC_BAD_ARGS (-2)     // misaligned / non-multiple-of-8 sizes
#define TPB_NOALLOC_NO_SYMBOL (-23)   // the device address of the scratch could not be obtained

#ifdef __cplusplus
extern "C" {
#endif

// RMSNorm backward without any allocation. Same math and argument meaning as tpb_rmsnorm_bwd:
//   dx = rstd * (w * dy - xhat * mean(w * dy * xhat)) [+ dres],   dw = sum_rows dy * xhat
// dy, x, dx: bf16 [rows, H] with the given row strides (elements); w: bf16 [H]; rstd: fp32 [rows];
// dres: optional bf16 [rows, H] (contiguous); dw_f32 / dw_bf16: either may be null;
// dw_accumulate != 0 adds to the existing dw. Returns 0, a negative TPB_NOALLOC_* code, or a
// positive cudaError_t from the launch.
int tpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                            const void* dres, void* dx, float* dw_f32, void* dw_bf16,
                            int dw_accumulate, int rows, int H, long long x_stride,
                            long long dy_stride, long long dx_stride, void* stream);

// Human-readable text for the codes above (and "ok" / "CUDA error" otherwise).
const char* tpb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
