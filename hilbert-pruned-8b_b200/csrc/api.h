// C interface of the kernel library (loaded from Python with ctypes).
//
// Conventions: pointers are device pointers unless named host_*; `stream` is a cudaStream_t;
// dtypes are HbDtype codes (0 = float32, 1 = bfloat16); row-major matrices with explicit row
// strides in elements; every function returns 0 or sets hb_last_error().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* hb_last_error(void);
int hb_device_info(int device, int* sm_major, int* sm_minor, int* sm_count);

// `status` (here and below): the caller's int32[4] status words (common.cuh: a bounded wait that
// ran out, non-finite logits, a bad page number, a bad token id), or null.
// `packed`: the table is stored as contiguous 128 x 64 tiles (the layout of hb_gemm_tc's packed weights)
int hb_embed(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens, int hidden,
             int vocab, int packed, int* status, void* stream);
int hb_rmsnorm(const float* x, const float* weight, float eps, float offset, void* out, int out_dtype,
               const int* rows, int n_rows, int hidden, void* stream);
int hb_silu_mul(const void* gate_up, int in_dtype, long long in_stride, void* out, int out_dtype,
                long long out_stride, int n_rows, int inter, void* stream);
int hb_rope_table(const int* positions, const float* inv_freq, float* out, int n_tokens, int half, void* stream);
int hb_rope_kv_append(void* qkv, int qkv_dtype, long long qkv_stride, const float* table, int rot,
                      int n_heads, int n_kv_heads, int head_dim, void* k_cache, void* v_cache, int cache_dtype,
                      const int* page_table, int pt_width, const int* tok_seq, const int* positions,
                      int n_tokens, int append, int n_pages, int* status, void* stream);
// Time marks of a timeline build (see common.cuh); other builds refuse.
int hb_timeline_set(void* marks, void* count, int capacity, int events);
int hb_gemm_general(const void* a, int a_dtype, long long lda, const void* w, int w_dtype, long long ldw,
                    void* out, int out_dtype, long long ldc, int M, int N, int K, int accumulate, void* stream);
int hb_gemm_tc_token_tile(int M);
long long hb_gemm_tc_scratch_floats(int M, int N, int K, int mode, int schedule);
long long hb_gemm_tc_tiles(int M, int N, int mode);
int hb_gemm_tc_resident_clusters(int mode, int size);
int hb_gemm_tc(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
               int M, int N, int K, int mode, int up_row0, int schedule, float* partials, long long partials_capacity,
               int* tile_counters, long long counters_capacity, int* error_flag, int packed, void* stream);
// A norm between two products, folded into them (hb_gemm_tc_fold; null pointers: that side is not used).
typedef struct {
    const float* prep_w;        // producer (mode 2): the norm's weight; the factor is prep_offset + prep_w[feature]
    float prep_offset;
    void* prep_out;             // bfloat16 [M, prep_ld]: the new residual values times the factor
    long long prep_ld;
    float* prep_sumsq;          // [M, sumsq_ld]: per token, the sums of squares of each 32 features
    const float* scale_sumsq;   // consumer (modes 0, 1, 3): such sums, written by the producer
    int scale_parts;            // how many of them per token
    float scale_inv_size;       // 1 / (features of the normed vector)
    float scale_eps;
    int sumsq_ld;
} HbNormFold;
int hb_gemm_tc_fold(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
               int M, int N, int K, int mode, int up_row0, int schedule, float* partials, long long partials_capacity,
               int* tile_counters, long long counters_capacity, int* error_flag, int packed, const HbNormFold* fold, void* stream);
int hb_gemm_tc2_wanted(int M, int N, int K);
int hb_gemm_tc2_resident_pairs(int mode);
int hb_gemm_tc2(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out, long long ldc,
                int M, int N, int K, int mode, int up_row0, int* error_flag, int packed, void* stream);
int hb_attention_general(const void* q, int q_dtype, long long q_stride, const void* k_cache, const void* v_cache,
                         int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                         const int* positions, void* out, int out_dtype, long long out_stride, int n_tokens,
                         int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_pages, int* status,
                         void* stream);
int hb_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_decode_ctas_per_sm(int head_dim);
long long hb_attention_decode_scratch_floats(int batch, int n_heads, int head_dim, int splits);
int hb_attention_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                        const int* page_table, int pt_width, const int* positions, float* scratch, void* out,
                        long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim, float scale,
                        int window, int splits, int max_pages, int n_pages, int* status, void* stream);
int hb_attention_decode_combined(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                 const int* page_table, int pt_width, const int* positions, float* scratch, int* counters,
                                 void* out, long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                 float scale, int window, int splits, int max_pages, int n_pages, int* status,
                                 void* stream);
int hb_attention_decode_fused(const void* qkv, long long stride, const float* table, int rot, void* k_cache,
                              void* v_cache, const int* page_table, int pt_width, const int* positions, float* scratch,
                              int* counters, void* out, long long out_stride, int batch, int n_heads, int n_kv_heads,
                              int head_dim, float scale, int window, int splits, int max_pages, int n_pages, int append,
                              int* status, void* stream);
int hb_attention_prefill_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                         const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0, void* out,
                         long long out_stride, int n_seqs, int q_blocks, int n_heads, int n_kv_heads, int head_dim,
                         float scale, int window, int n_pages, int* status, void* stream);
int hb_attention_prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim);
int hb_attention_prefill_tc(const void* q, long long q_stride, long long n_tokens, const void* k_cache, const void* v_cache,
                            const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0, void* out,
                            long long out_stride, int n_seqs, int q_blocks, int n_heads, int n_kv_heads, int head_dim,
                            float scale, int window, int n_pages, int* error_flag, void* stream);
// out[i] = mean + stdev * N(0, 1): element i of the counter-based stream `base`
int hb_random_normal(void* out, int out_dtype, long long n, unsigned long long base, float stdev, float mean,
                     void* stream);
int hb_argmax(const float* logits, long long stride, int* out, int n_rows, int vocab, int parts, void* scratch,
              int* counters, int* status, void* stream);
int hb_sample(const float* logits, long long stride, const float* temperature, const long long* seeds,
              const long long* request_ids, const long long* steps, int* out, int n_rows, int vocab, int* status,
              void* stream);

#ifdef __cplusplus
}
#endif
