// The C interface of the kernel library.  Every function launches on `stream`, allocates
// nothing and returns 0, a cudaError_t value, or one of the WPC_ERR_* codes of common.cuh.
// Element types are named by WPC_DTYPE_F32 (0) and WPC_DTYPE_BF16 (1).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Programmatic dependent launch for all kernels of the library: on (1, the default) or off (0).
int wpc_set_pdl(int on);
// How long a kernel waits on one of its mbarriers before it gives up, records
// WPC_ERR_DEVICE_WAIT in the status word it was given and returns (default 2 s).  `starve` = 1
// is for tests of that path: the kernels with TMA producers start no copies, so their waits
// run out; nothing else about them changes.
int wpc_set_wait_policy(unsigned long long limit_ns, int starve);

int wpc_embed(const int* tokens, const void* table, int table_dtype, float* out, int T, int H, int V,
              cudaStream_t stream);
// rows == null: out [T, H]; else out [n_rows, H], row i the norm of x[rows[i]]
int wpc_rmsnorm(const float* x, const float* gain, float eps, void* out, int out_dtype, int T, int H,
                const int* rows, int n_rows, cudaStream_t stream);
// out[t, i] = act(gate) * up; act: WPC_ACT_SILU (1) or WPC_ACT_GELU_TANH (2) of common.cuh
int wpc_gate_mul(const void* gu, void* out, int dtype, int T, int I, int group, int act, cudaStream_t stream);
int wpc_add(float* x, const void* y, int y_dtype, size_t n, cudaStream_t stream);
int wpc_gather_rows(const float* x, const int* idx, float* out, int n_rows, int H, int T, cudaStream_t stream);
int wpc_convert(const void* in, int in_dtype, void* out, int out_dtype, size_t n, cudaStream_t stream);
int wpc_rope_angles(const int* positions, const double* inv_freq, float* cosv, float* sinv, int T, int R,
                    cudaStream_t stream);
// interleaved = 0: pairs (r, r + hd/2); 1: pairs (2r, 2r + 1)
int wpc_rope_inplace(void* x, int dtype, int row_stride, int T, int n_heads, int hd, int R, const float* cosv,
                     const float* sinv, int interleaved, cudaStream_t stream);
// RMS norm with gain [hd] of each of the first n_heads heads of every row, in place
int wpc_head_rmsnorm(void* x, int dtype, int row_stride, int T, int n_heads, int hd, const float* gain, float eps,
                     cudaStream_t stream);
int wpc_qk_rope_kv_store(void* qkv, int dtype, int row_stride, int T, int nh, int nkv, int hd, int R,
                         const float* cosv, const float* sinv, void* k_pages, void* v_pages,
                         const int* page_table, int table_width, const int* seq_of_token, const int* positions,
                         int n_pages, int* status, cudaStream_t stream);
int wpc_fill_normal(void* out, int dtype, size_t n, uint64_t key, float mean, float std, cudaStream_t stream);

int wpc_gemm_simt(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw, const float* bias,
                  void* C, int out_dtype, int ldc, int accumulate, int M, int N, int K, cudaStream_t stream);

int wpc_gemm_tc_set_stage_limit(int limit);
int wpc_gemm_tc_workspace(int rows_a, int rows_b, int bn, int splits, size_t* scratch_floats, int* n_counters);
int wpc_gemm_tc(const void* a, int lda, int rows_a, const void* b, int ldb, int rows_b, int K, const float* bias,
                void* out, int out_dtype, int ldc, int accumulate, int gated, int swap, int bn, int splits,
                float* scratch, size_t scratch_floats, int* counters, int n_counters, int* status,
                int prefetch_weights, int tall, int cluster, cudaStream_t stream);
int wpc_gemm_tc_cluster_capacity(int bn, int splits);
int wpc_gemm_tc_rope_store(const void* w, int ldw, const void* x, int ldx, int tokens, int K, const float* bias, void* out,
                           int ldc, int bn, int splits, int prefetch_weights, int nh, int nkv, int hd, int R,
                           const float* cosv, const float* sinv, void* k_pages, void* v_pages, const int* page_table,
                           int table_width, const int* seq_of_token, const int* positions, int n_pages, int* status,
                           cudaStream_t stream);

int wpc_attention_plain(const void* q, int q_stride, void* out, int out_stride, int dtype, const void* k_pages,
                        const void* v_pages, const int* page_table, int table_width, const int* seq_of_token,
                        const int* positions, int T, int nh, int nkv, int hd, float scale, int window,
                        int n_splits, float* part, cudaStream_t stream);

int wpc_attention_mma_supports(int nh, int nkv, int hd);
int wpc_attention_decode_early_pages(int on);
int wpc_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                         const void* v_pages, const int* page_table, int table_width, const int* ctx_lens, int B,
                         int nh, int nkv, int hd, float scale, int window, int n_ctas, float* part_o, float* part_ml,
                         int* counters, int n_counters, cudaStream_t stream);
int wpc_attention_decode_cluster_capacity(int hd, int cluster, int alone);
int wpc_attention_decode_cluster(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                 const void* v_pages, const int* page_table, int table_width, const int* ctx_lens,
                                 int B, int nh, int nkv, int hd, float scale, int window, int cluster, int groups,
                                 float* part_o, float* part_ml, int* counters, int n_counters,
                                 cudaStream_t stream);
int wpc_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                          const int* ctx_lens, int B, int max_new, int nh, int nkv, int hd, float scale, int window,
                          cudaStream_t stream);

int wpc_attention_prefill_tc_supports(int nh, int nkv, int hd);
int wpc_attention_prefill_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                             const void* v_pages, const int* page_table, int table_width, const int* cu_seqlens,
                             const int* ctx_lens, int B, int max_new, int nh, int nkv, int hd, float scale,
                             int window, int* status, int n_pages, int tiles, cudaStream_t stream);

int wpc_sample(const float* logits, int n_rows, int V, const int* slots, long long* seq_state, float temperature,
               const int* banned, int n_banned, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
