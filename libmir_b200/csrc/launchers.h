// Prototypes of the exported launchers that other translation units of the same library call (the layer executor
// and the bfloat16 product dispatch).  Every launcher returns a MirStatus and leaves its text in mir_last_error().
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

extern "C" {
// elementwise.cu
int mir_rms_norm(int bf16, const float* x, const float* weight, void* out, const int* rows, int n_rows, int hidden,
                 float eps, cudaStream_t stream);
int mir_silu_mul(int bf16, const void* gate_up, void* out, int rows, int inter, cudaStream_t stream);
int mir_add_bias(int bf16, float* x, const void* bias, int rows, int cols, cudaStream_t stream);
// qk_rope_store.cu
int mir_qk_rope_store(int bf16, void* qkv, const int* positions, const int* slot_mapping, const float* inv_freq,
                      const float* q_norm, const float* k_norm, void* k_pages, void* v_pages, int tokens, int heads,
                      int kv_heads, int head_dim, int rotary_dim, float eps, int write_kv, cudaStream_t stream);
// attention_generic.cu
int mir_paged_attention_generic(int bf16, const void* q, long long q_token_stride, void* out, const void* k_pages,
                                const void* v_pages, const int* block_table, int table_width, const int* row_of_token,
                                const int* positions, int tokens, int page_size, int heads, int kv_heads, int head_dim,
                                float scale, int window, cudaStream_t stream);
// gemm_f32.cu
int mir_gemm_f32(const float* a, int lda, const float* w, int ldw, const float* bias, float* c, int ldc, int m, int n,
                 int k, float beta, cudaStream_t stream);
#ifdef MIR_WITH_BF16
// gemm_lt.cu, gemm_tc_stream.cu, gemm_tc.cu
int mir_gemm_bf16_lt(const void* x, int ldx, const void* w, int ldw, const void* bias, void* out, int ldo, int out_f32,
                     int m, int n, int k, float beta, void* workspace, size_t workspace_bytes, cudaStream_t stream);
int mir_gemm_tc_stream_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m,
                            int n, int k, int up_offset, const float* sumsq, int sumsq_tiles, float eps,
                            float* sumsq_out, const float* next_weight, void* weighted_out, int ld_weighted,
                            cudaStream_t stream);
int mir_gemm_tc_stream_head_candidates(int n);
int mir_gemm_tc_stream_head_bf16(const void* x, int ldx, const void* w, void* out, int ldo, int m, int n, int k,
                                 float* best_value, int* best_index, int best_stride, cudaStream_t stream);
int mir_gemm_tc_bf16(int mode, const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int m, int n,
                     int k, int up_offset, cudaStream_t stream);
// attention_mma.cu, attention_tc.cu, attention_tc_decode.cu
long long mir_decode_attention_scratch_floats(int rows, int heads, int head_dim, int num_partitions);
int mir_decode_attention_bf16(const void* q, long long q_stride, void* out, const void* k_pages, const void* v_pages,
                              const int* block_table, int table_width, const int* positions, int rows, int page_size,
                              int heads, int kv_heads, int head_dim, float scale, int window, int partition,
                              int num_partitions, float* scratch, long long scratch_floats, cudaStream_t stream);
int mir_decode_merge_bf16(const float* partial_o, const float* partial_ml, const int* positions, int rows, int heads,
                          int head_dim, int window, int partition, int num_partitions, void* out, cudaStream_t stream);
int mir_decode_attention_tc_takes(int head_dim, int page_size, int partition);
int mir_decode_attention_tc_bf16(const void* q, long long q_stride, void* out, const void* k_pages, const void* v_pages,
                                 long long cache_rows, const int* block_table, int table_width, const int* positions,
                                 int rows, int page_size, int heads, int kv_heads, int head_dim, float scale, int window,
                                 int partition, int num_partitions, float* scratch, long long scratch_floats,
                                 cudaStream_t stream);
int mir_prefill_attention_bf16(const void* q, long long q_stride, void* out, const void* k_pages, const void* v_pages,
                               const int* block_table, int table_width, const int* query_starts,
                               const int* context_lens, int num_rows, int tokens, int page_size, int heads,
                               int kv_heads, int head_dim, float scale, int window, cudaStream_t stream);
int mir_prefill_attention_tc_takes(int head_dim, int page_size);
int mir_prefill_attention_tc_bf16(const void* q, long long q_stride, void* out, const void* k_pages, const void* v_pages,
                                  long long cache_rows, const int* block_table, int table_width,
                                  const int* query_starts, const int* context_lens, int num_rows, int tokens,
                                  int page_size, int heads, int kv_heads, int head_dim, float scale, int window,
                                  cudaStream_t stream);
// ops_bf16.cu
int mir_linear_bf16(const void* x, int ldx, const void* w, const void* bias, void* out, int ldo, int out_f32,
                    int accumulate, int m, int n, int k, const float* sumsq, int sumsq_tiles, float eps,
                    float* sumsq_out, const float* next_weight, void* weighted_out, int ld_weighted, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream, int* wrote_stats);
int mir_gate_up_silu_bf16(const void* x, int ldx, const void* w_gate_up, void* out, int m, int inter, int k,
                          const float* sumsq, int sumsq_tiles, float eps, void* gate_up_scratch, void* workspace,
                          size_t workspace_bytes, cudaStream_t stream);
int mir_decode_attention_paged_bf16(const void* q, long long q_stride, void* out, const void* k_pages,
                                    const void* v_pages, long long cache_rows, const int* block_table, int table_width,
                                    const int* positions, int rows, int page_size, int heads, int kv_heads,
                                    int head_dim, float scale, int window, int partition, int num_partitions,
                                    float* scratch, long long scratch_floats, cudaStream_t stream);
int mir_decode_partition_keys(int rows, int heads, int kv_heads, int head_dim, int page_size, int longest);
int mir_decode_attention_plan(int rows, int heads, int kv_heads, int head_dim, int page_size, int longest,
                              int* partition, int* partitions, long long* scratch_floats);
int mir_get_option(const char* name);
#endif
}

// A folded norm's rows were given to a product that cannot take them over: the caller runs the norm as a kernel
// and calls again with the normed rows.
#define MIR_CANNOT_FOLD 4
