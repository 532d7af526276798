// Every entry point of the library, as C prototypes.  Each launcher takes raw device pointers and a stream,
// checks its sizes on the host and returns 0, a negative PE_ERR_* code for a size or argument it refuses
// (common.cuh), or a positive CUDA runtime error number.  kernels/lib.py declares the same signatures for
// ctypes; every .cu file includes this header, so a definition that drifts from it does not compile.
// pe_attention_decode_noalloc is described in attention_noalloc.h.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif


// attention_generic.cu
long long pe_attention_generic_scratch_floats(int n_seqs, int n_heads, int head_dim, int max_splits);
int pe_attention_generic(int dtype, int decode, const void* q, long long q_ld, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart,
    const int* seq_past, const int* seq_slot, const int* page_table, int table_stride, int num_pages,
    const void* k_pages, const void* v_pages, float* scratch, int split_keys, int max_splits, int* status,
    cudaStream_t stream);
int pe_attention_decode_noalloc(int dtype, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, int split_keys, int max_splits, int* status, cudaStream_t stream);

// attention_mma.cu
int pe_attention_mma_decode_blocks_per_sm(int head_dim);
int pe_attention_mma_supported(int head_dim, int n_heads, int n_kv_heads);
int pe_attention_mma(int decode, const void* q, long long q_ld, void* out, long long out_ld, int n_seqs, int max_q,
    int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart, const int* seq_past,
    const int* seq_slot, const int* page_table, int table_stride, int num_pages, const void* k_pages,
    const void* v_pages, float* scratch, int split_keys, int max_splits, int min_range_keys, int* status,
    cudaStream_t stream);

// attention_umma.cu
int pe_attention_umma_supported(int head_dim, int n_heads, int n_kv_heads);
int pe_attention_umma_prefill(const void* q, long long q_ld, long long n_tokens, void* out, long long out_ld,
    int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale, int window, const int* seq_qstart,
    const int* seq_past, const int* seq_slot, const int* page_table, int table_stride, int num_pages,
    const void* k_pages, const void* v_pages, int n_sms, int* work_counter, int* status, cudaStream_t stream);

// embedding.cu
int pe_embed_gather(int dtype, const void* table, const int* ids, float* out, int n_tokens, int hidden, int vocab,
    int* status, cudaStream_t stream);

// gemm_smallm.cu
int pe_gemm_smallm_supported(int M, int N, int K);
int pe_gemm_smallm(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, cudaStream_t stream);

// gemm_umma.cu
int pe_gemm_umma_supported(int M, int N, int K, int pair_offset);
int pe_gemm_umma(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream);

// gemm_umma2.cu
int pe_gemm_umma2_supported(int M, int N, int K, int pair_offset);
int pe_gemm_umma2(const void* x, long long ldx, const void* w, void* y, long long ldy, int M, int N, int K,
    int out_f32, int pair_offset, int n_sms, int* status, cudaStream_t stream);
int pe_gemm_umma2_qkv_rope_supported(int M, int K, int n_heads, int n_kv_heads, int head_dim, int rotary_dim);
int pe_gemm_umma2_qkv_rope(const void* x, long long ldx, const void* w, void* qkv, long long ld, int M, int K,
    int n_heads, int n_kv_heads, int head_dim, const float* q_norm_w, const float* k_norm_w, float eps,
    const float* cos_table, const float* sin_table, int rotary_dim, int table_rows, const int* token_seq,
    const int* token_pos, const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride,
    int num_pages, void* k_pages, void* v_pages, int write_cache, int n_sms, int* status, cudaStream_t stream);

// rmsnorm.cu
int pe_rmsnorm_residual(int dtype, float* residual, const void* delta, const float* weight, void* out,
    const int* rows, int n_rows, int dim, float eps, cudaStream_t stream);
int pe_rmsnorm(int dtype, const void* x, const float* weight, void* out, int n_rows, int dim, float eps,
    cudaStream_t stream);

// rope_append.cu
int pe_batch_expand(const int* seq_qstart, const int* seq_past, int n_seqs, int* token_seq, int* token_pos,
    cudaStream_t stream);
int pe_qk_norm_rope_append(int dtype, void* qkv, long long ld, int n_tokens, int n_heads, int n_kv_heads,
    int head_dim, const float* q_norm_w, const float* k_norm_w, float eps, const float* cos_table,
    const float* sin_table, int rotary_dim, int table_rows, const int* token_seq, const int* token_pos,
    const int* seq_slot, const int* seq_qstart, const int* page_table, int table_stride, int num_pages,
    void* k_pages, void* v_pages, int write_cache, int* status, cudaStream_t stream);

// sampling.cu
long long pe_sample_scratch_bytes(int n_rows, int vocab, float temperature, int top_k, float top_p, float min_p);
int pe_sample(const float* logits, long long ld, int n_rows, int vocab, float temperature, int top_k, float top_p,
    float min_p, unsigned long long seed, const int* row_request, const int* row_step, int* out_tokens,
    void* scratch, long long scratch_bytes, cudaStream_t stream);
int pe_repetition_penalty(float* logits, long long ld, int n_rows, int vocab, const int* recent, int recent_stride,
    const int* recent_count, float penalty, cudaStream_t stream);

// swiglu.cu
int pe_silu_mul(int dtype, const void* gate_up, void* out, int n_rows, int inter, cudaStream_t stream);

// wait_probe.cu
int pe_wait_probe(unsigned long long* out, int polls, cudaStream_t stream);
long long pe_wait_limit_polls();

#ifdef __cplusplus
}
#endif
