// C ABI of libtpb200 (the sm_100a kernel library). Every entry point takes raw device
// pointers plus the CUDA stream to launch on, returns 0 on success, a negative value for
// rejected arguments and a positive cudaError_t / CUresult otherwise. None of them allocates
// device memory; scratch buffers are passed in by the caller.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
namespace tpb {
int sm_count();
void ensure_thread_context();
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t ld,
                      uint32_t box1);
int make_tmap_2d_u8(CUtensorMap* out, const void* base, uint64_t d0, uint64_t d1, uint64_t ld,
                    uint32_t box1);
int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                   const uint64_t* strides_elems, const uint32_t* box, int swizzle128);
// Mapped symmetric arenas of this process (see symm_comm.cu); null before tpb_symm_create.
struct SymmView {
  int world, rank;
  char* peer[16];
};
const SymmView* symm_view();
// Optional fused-collective description handed to the GEMM (see GemmParams in gemm_tcgen05.cu).
struct GemmFused {
  int n_copy, ag_operand, world, rank;
  const char* ag_src[16];
  char* ag_dst;
  unsigned long long ag_shard_bytes, ag_chunk_bytes;
  int ag_rows_per_rank, ag_rows_per_flag;
  uint32_t* ag_flags;
  uint32_t* pad_local;
  uint32_t* pad_peer[16];
  int ready_slot, done_slot;
  uint32_t epoch;
  const uint32_t* epoch_dev;  // device-side epoch word (epoch = *epoch_dev + 1) or null
  uint32_t rs_per_call;
  int tile_m_shift;
  int tile_n_shift;
  int rs_mode, rs_rows_per_rank;
  char* rs_stage[16];
  uint32_t* rs_cnt[16];
  uint32_t rs_expect;
  __nv_bfloat16* rs_out;
  unsigned long long wait_ns;
};
// The registered split-K workspace (null when none): fp32 partial tiles and one flag per tail tile.
void splitk_workspace(float** ws, uint32_t** flags);
int gemm_pair_dispatch(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                       int ldb, int ldc, int a_mn, int b_mn, int out_f32, int bias_f32, int accumulate,
                       float alpha, int max_ctas, uint32_t* status, cudaStream_t stream, int block_n = 0);
int gemm_bf16_dispatch(const void* A, const void* B, void* C, const void* bias, int M, int N,
                       int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32,
                       int bias_f32, int accumulate, float alpha, const uint32_t* b_flags,
                       int rows_per_flag, uint32_t flag_want, int max_ctas, uint32_t* status,
                       cudaStream_t stream, const GemmFused* fused);
}  // namespace tpb
extern "C" {
#endif

// C[m,n] (+)= alpha * sum_k A(m,k) B(n,k) (+ bias[n]); bf16 operands, fp32 accumulate.
//   a_mn = 0: A is [M, K] row-major (lda elements per row); a_mn = 1: A is stored [K, M].
//   b_mn = 0: B is [N, K] row-major;                         b_mn = 1: B is stored [K, N].
//   status: device word, receives a tpb status code if a bounded wait gives up.
int tpb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                  int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32, int bias_f32,
                  int accumulate, float alpha, uint32_t* status, void* stream);

long long tpb_gemm_splitk_workspace_bytes();
int tpb_gemm_set_splitk_workspace(void* ws, uint32_t* flags);

int tpb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out,
                    float* rstd, int rows, int H, long long x_stride, long long y_stride,
                    float eps, void* stream);
int tpb_rmsnorm_bwd_grid(int rows, int H);
int tpb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                    const void* dres, void* dx, float* dw_part, float* dw_f32, void* dw_bf16,
                    int dw_accumulate, int rows, int H, long long x_stride, long long dy_stride,
                    long long dx_stride, void* stream);
int tpb_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                      float* rstd, int rows, int H, float eps, void* stream);
int tpb_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                      const float* rstd, void* dx, float* dw_part, float* db_part, float* dw_f32,
                      void* dw_bf16, float* db_f32, void* db_bf16, int accumulate, int rows, int H,
                      void* stream);
int tpb_rope(void* x, const float* cos_t, const float* sin_t, const long long* pos,
             long long tokens, int heads, int D, long long tok_stride, long long head_stride,
             int seq_len, int interleaved, int backward, void* stream);
int tpb_rope_out(const void* x, void* y, const float* cos_t, const float* sin_t, const long long* pos,
                 long long tokens, int heads, int D, long long tok_stride, long long head_stride,
                 long long y_tok_stride, long long y_head_stride, int seq_len, int interleaved,
                 int backward, void* stream);
int tpb_swiglu_fwd(const void* gate, const void* up, void* out, long long rows, int I,
                   long long in_stride, void* stream);
int tpb_swiglu_bwd(const void* dy, const void* gate, const void* up, void* dgate, void* dup,
                   long long rows, int I, long long in_stride, long long out_stride, void* stream);
int tpb_gelu_fwd(const void* x, void* y, long long n, int approx, void* stream);
int tpb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, int approx, void* stream);
int tpb_cross_entropy(const void* logits, const long long* target, float* loss, float* lse,
                      void* dlogits, long long rows, int V, long long stride,
                      long long ignore_index, float gscale, void* stream);

int tpb_cross_entropy_bwd(const void* logits, const long long* target, const float* lse,
                          void* dlogits, const float* g_scalar, const float* scale,
                          const float* g_rows, long long rows, int V, long long stride,
                          long long ignore_index, void* stream);

int tpb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Tq,
                  int Tk, int Hq, int Hkv, int D, long long q_tok, long long q_head,
                  long long q_batch, long long k_tok, long long k_head, long long k_batch,
                  long long v_tok, long long v_head, long long v_batch, long long o_tok,
                  long long o_head, long long o_batch, int lse_stride, int causal, float scale,
                  uint32_t* status, void* stream, const int* kv_len, int n_splits,
                  long long o_split_stride, long long lse_split_stride);
int tpb_flash_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
                  const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int Tq,
                  int Tk, int Hq, int Hkv, int D, long long q_tok, long long q_head,
                  long long q_batch, long long k_tok, long long k_head, long long k_batch,
                  long long v_tok, long long v_head, long long v_batch, long long o_tok,
                  long long o_head, long long o_batch, long long do_tok, long long do_head,
                  long long do_batch, long long dq_tok, long long dq_head, long long dq_batch,
                  long long dkv_tok, long long dkv_head, long long dkv_batch, int lse_stride,
                  int causal, float scale, uint32_t* status, void* stream);

int tpb_grouped_workspace_ints(int max_rows, int G);
int tpb_grouped_gemm(const void* A, const void* B, void* C, const int* offs, int G, int max_rows,
                     int N, int K, int mode, int b_mn, int out_f32, int accumulate, int* workspace,
                     uint32_t* status, void* stream);

int tpb_adamw_flat(float* master, float* m, float* v, const void* grad, int grad_bf16, void* model,
                   int model_bf16, long long n, float lr, float beta1, float beta2, float eps,
                   float wd, int step, float grad_scale, int maximize, const float* clip_coef,
                   const float* found_inf, void* stream);
int tpb_adamw_multi(int count, void* const* master, void* const* m, void* const* v,
                    const void* const* grad, void* const* model, const long long* numel,
                    int grad_bf16, int model_bf16, float lr, float beta1, float beta2, float eps,
                    float wd, int step, float grad_scale, int maximize, const float* clip_coef,
                    const float* found_inf, void* stream);
int tpb_sumsq(const void* x, int is_bf16, long long n, float scale, float* out, void* stream);
int tpb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, void* stream);

#ifdef __cplusplus
}
#endif
