// Public C ABI of libscirust_b200_cuda.so: every extern "C" entry point of csrc/*.cu, declared once.
// Python reaches these through ctypes (scirust_b200/ops/_lib.py and the ops modules' register() calls); every
// entry point takes raw device pointers plus the CUDA stream to launch on, allocates nothing unless stated, and
// returns 0 or an SB_ERR_* code. The declarations below the marker are generated from the definitions
// (python -m scirust_b200._build --api-header); a test compares them with the sources and with the ctypes tables.
// Kernels that can wait (mbarrier / peer flags) also take a device `status` word: they store an sb::ST_* code
// there when a bounded wait runs out.
#pragma once
#include <stddef.h>
#include <stdint.h>

#define SB_ERR_ARG 1
#define SB_ERR_ALIGN 2
#define SB_ERR_DRIVER 3
#define SB_ERR_LAUNCH 4
#define SB_ERR_TOO_LARGE 5
#define SB_ERR_RUNTIME 6

#ifdef __cplusplus
extern "C" {
#endif

// ---- entry points (generated from the definitions by scirust_b200._build.write_api_header) ----

// attention_bwd_tcgen05.cu
size_t sb_attention_bwd_ds_elems(int B, int S, int H);
int sb_attention_bwd(const void* qkv, const void* O, const float* lse, const void* dO, void* dqkv, float* delta, void* ds_scratch, int B, int S, int H, int Hkv, int dh, int ld, int ld_o, int ld_do, float scale, int causal, int* status, void* stream_);

// attention_fwd_pp_tcgen05.cu
int sb_attention_fwd_pp(const void* qkv, void* O, float* lse, int B, int S, int H, int Hkv, int dh, int ld, int ld_o, float scale, int causal, int* status, void* stream_);

// attention_fwd_tcgen05.cu
int sb_attention_fwd(const void* qkv, void* O, float* lse, int B, int S, int H, int Hkv, int dh, int ld, int ld_o, float scale, int causal, int* status, void* stream_);

// canonical_strict.cu
int sb_canon_elementwise(int op, const void* a, const void* b, void* out, long long n, uint32_t factor_bits, void* stream_);
int sb_canon_permute(const void* in, void* out, int rank, const long long* in_shape, const int* perm, void* stream_);

// comm.cu
int sb_malloc(size_t bytes, void** out);
int sb_free(void* p);
int sb_memset(void* p, int v, size_t bytes, void* stream);
int sb_ipc_get_handle(void* p, void* handle_out);
int sb_ipc_open(const void* handle, void** out);
int sb_ipc_close(void* p);
int sb_ipc_handle_size();
int sb_flag_words_per_slot();
int sb_allreduce_bf16(void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank, int W, size_t n_elems, float scale, uint32_t epoch, int slot, int out_fp32, unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream);
int sb_allreduce_bf16_lean(void* const* in_ptrs, void* const* out_ptrs, void* const* flag_ptrs, int rank, int W, size_t n_elems, float scale, uint32_t epoch, int slot, int out_fp32, unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream);
int sb_small_collective(void* const* in_ptrs, void* const* flag_ptrs, int rank, int W, int mode, int in_fp32, size_t n, int rows, const void* residual, void* out, uint32_t* epoch_word, int slot, unsigned int* cta_counter, int n_ctas, int wait_ms, int* status, void* stream);
int sb_wait_probe(const void* flags, int W, uint32_t epoch, int wait_ms, int* status, void* stream);

// conv.cu
int sb_im2col_nhwc(const void* x, void* col, int B, int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW, int Kp, void* stream);
int sb_col2im_nhwc(const void* dcol, void* dx, int B, int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW, int Kp, void* stream);
int sb_maxpool_fwd(const void* x, void* y, void* arg, int B, int H, int W, int C, int k, int stride, int OH, int OW, void* stream);
int sb_maxpool_bwd(const void* dy, const void* arg, void* dx, int B, int H, int W, int C, int k, int stride, int OH, int OW, void* stream);
int sb_colstats(const void* a, const void* b, float* partial, float* s1, float* s2, int rows, int C, void* stream);
int sb_bn_fwd(const void* x, const float* sum, const float* sumsq, const float* gamma, const float* beta, float* mean, float* inv_std, float* run_mean, float* run_var, void* y, int rows, int C, float eps, float momentum, int relu, int training, void* stream);
int sb_bn_bwd(const void* g, const void* x, const float* sum_g, const float* sum_gx, const float* mean, const float* inv_std, const float* gamma, float* dgamma, float* dbeta, void* dx, int rows, int C, void* stream);
int sb_relu_mask(const void* dy, const void* y, void* g, size_t total, void* stream);
int sb_bias_act(const void* x, const float* bias, void* y, size_t total, int C, int relu, void* stream);

// decode.cu
int sb_set_pdl(int on);
int sb_gemv(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R, int ldr, void* out_bf16, int ldo, float* out_f32, int M, int N, int K, int is_int8, int splits, float* workspace, int prologue, const void* norm_w, float eps, int* status, void* stream);
int sb_gemv_allreduce(const void* X, int ldx, const void* W, int ldw, const float* scale, const void* R, int ldr, void* out_bf16, int ldo, int M, int N, int K, int is_int8, int splits, float* workspace, int prologue, const void* norm_w, float eps, void* const* recv_ptrs, void* const* flag_ptrs, uint32_t* epoch_word, unsigned int* done_ctr, int rank, int world, int rows, int wait_ms, int* status, void* stream);
int sb_gemv_argmax(const void* X, int ldx, const void* W, int ldw, const float* scale, float* logits_f32, int M, int N, int K, int is_int8, int splits, float* workspace, int prologue, const void* norm_w, float eps, int32_t* amax_ws, int64_t* out_tokens, int64_t* generated, int gen_stride, int step, int col_offset, void* const* cand_ptrs, void* const* flag_ptrs, uint32_t* epoch_word, int rank, int world, int wait_ms, int* status, void* stream);
int sb_kv_append(const void* qkv, int ld, int H, int Hkv, int dh, void* pool, const int* block_table, int max_blocks, int page, const int* seq_of, const int* pos, int n_tok, void* stream);
int sb_rope_kv_append(void* qkv, int ld, int H, int Hkv, int dh, const float* cos_t, const float* sin_t, void* pool, const int* block_table, int max_blocks, int page, const int* seq_of, const int* pos, int n_tok, void* stream);
int sb_decode_attention(const void* q, int ldq, const void* pool, const int* block_table, int max_blocks, int page, const int* seq_len, int B, int H, int Hkv, int dh, int n_splits, float scale, float* part_o, float* part_ml, unsigned int* counters, void* out, int ldo, void* stream);
int sb_argmax(const float* logits, int rows, int V, float* pval, int* pidx, int64_t* out_tokens, int64_t* generated, int gen_stride, int step, void* stream);
int sb_quantize_per_channel(const void* W, int K, int N, int ldw, float* scale, void* Q, void* stream);
int sb_dequantize(const void* Q, const float* scale, int K, int N, void* W, void* stream);

// gemm_dist_tcgen05.cu
int sb_gemm_dist_bf16(void* const* a_ptrs, void* const* b_ptrs, void* C, const void* R, void* const* stage_ptrs, void* const* flag_ptrs, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int a_gather, int b_gather, int scatter, int rank, int W, uint32_t epoch, unsigned int* counters, int bn, int wait_ms, void* a_stage, int ld_stage, uint32_t* chunk_flags, unsigned int* chunk_ctr, int* status, void* stream_);

// gemm_i8_tcgen05.cu
int sb_quantize_rows(const void* x, int ldx, void* xq, int ldq, float* sx, int M, int K, void* stream);
int sb_gemm_i8(const void* xq, int ldq, const float* sx, const void* wq_t, int ldw, const float* sw, void* C, int ldc, const void* R, int ldr, int M, int N, int K, int splits, void* workspace, int* status, void* stream);

// gemm_pair_tcgen05.cu
size_t sb_gemm_pair_workspace_floats();
int sb_gemm_pair_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, void* workspace, void* act, int ld_act, int ff, const void* gu, int ld_gu, int* status, void* stream_);
int sb_gemm_pair_ag_bf16(void* const* a_ptrs, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int b_mn, void* const* stage_ptrs, int ld_stage, void* const* flag_ptrs, void* const* chunk_flag_ptrs, unsigned int* chunk_ctr, unsigned int* cta_ctr, int rank, int W, uint32_t epoch, int wait_ms, int copy_own, int* status, void* stream_);
int sb_gemm_pair_rs_bf16(const void* A, const void* B, void* const* part_ptrs, int ldp, void* out, int ld_out, const void* res, int ld_res, int M, int N, int K, int lda, int ldb, int b_mn, void* const* ready_ptrs, void* const* flag_ptrs, unsigned int* block_ctr, unsigned int* cta_ctr, int rank, int W, uint32_t epoch, int wait_ms, int* status, void* stream_);

// gemm_skinny_tcgen05.cu
int sb_gemm_skinny(const void* X, int ldx, const void* W, int ldw, void* C, int ldc, const void* R, int ldr, int rows, int N, int K, int is_i8, const float* sx, const float* sw, int splits, void* workspace, int* status, void* stream_);

// gemm_tcgen05.cu
size_t sb_gemm_balanced_workspace_floats();
int sb_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int splits, void* workspace, int bn, int* status, void* stream_);

// gemm_w8_tcgen05.cu
int sb_gemm_w8(const void* A, const void* Q, const float* scale, void* C, const void* R, int M, int N, int K, int lda, int ldq, int ldc, int ldr, int splits, void* workspace, int* status, void* stream_);

// kernels_basic.cu
int sb_rmsnorm_fwd(const void* x, const void* w, void* y, float* inv_rms, int rows, int cols, int ldx, int ldy, float eps, void* stream);
int sb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* inv_rms, const void* dres, void* dx, float* dw_partial, float* dw_f32, void* dw_bf16, int rows, int cols, void* stream);
int sb_rope(void* x, int ld, int rows, int n_heads, int dh, int seq_len, int offset, const int* positions, const float* cos_t, const float* sin_t, int backward, void* stream);
int sb_swiglu_fwd(const void* gu, void* h, int rows, int ff, void* stream);
int sb_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int ff, void* stream);
int sb_add_bf16(const void* a, const void* b, void* out, size_t n, void* stream);
int sb_embed_fwd(const void* table, const int64_t* tokens, void* out, int n, int d, int vocab, void* stream);
int sb_embed_bwd(const void* dy, const int64_t* sorted_tok, const int64_t* perm, void* dtable, int n, int d, int vocab, int accumulate, void* stream);
int sb_ce_fwd_bwd(const void* logits, const int64_t* targets, float* loss_rows, void* dlogits, int rows, int cols, int ld, float grad_scale, void* stream);
int sb_ce_shard_stats(const void* logits, const int64_t* targets, float* stats, int rows, int cols, int ld, int v0, void* stream);
int sb_ce_shard_grad(const void* logits, const int64_t* targets, const float* lse, void* dlogits, int rows, int cols, int ld, int v0, float grad_scale, void* stream);
int sb_sumsq(const void* g, size_t n, int is_bf16, float* partials, float* out, int accumulate, void* stream);
int sb_optim_step(float* p, float* m, float* v, const void* grad, int grad_is_bf16, void* p_bf16, size_t n, size_t decay_end, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_sumsq, float max_grad_norm, float grad_scale, int mode, void* stream);
int sb_cast(const void* in, void* out, size_t n, int to_bf16, float scale, void* stream);
int sb_multi_cast_f32_bf16(const void* const* srcs, const unsigned long long* dst_offs, const unsigned long long* ns, int count, void* dst, int accumulate, void* stream);
int sb_sumsq_no_alloc(const void* g, size_t n, int is_bf16, float* out, int accumulate, void* stream);

// sampler.cu
int sb_sample_rows(const float* logits, int ld, int rows, int V, float temperature, int top_k, float top_p, float rep_penalty, int rep_window, const int64_t* recent, int recent_ld, const int* n_recent, uint64_t* rng_state, int64_t* out_tokens, int64_t* generated, int gen_stride, int step, uint32_t* work, void* stream);

// ---- end of entry points ----

#ifdef __cplusplus
}
#endif
