// General causal attention over the paged cache: any head size up to 256, any head and
// group count, float32 or bfloat16 cache, optional window.  One block per (token, query
// head).  It serves prefill and decode alike: the true 32-bit path uses it everywhere, the
// bfloat16 path wherever the specialised kernels refuse a size.
//
// Per query (cleanroom-transformer/src/cpu_backend.c:102-124; online form as in
// cuda_backend.cu:254-306): kv head g = j / (heads / kv_heads); keys lo..p with p the
// token's position and lo = max(0, p - window + 1); score = dot(q, k) * scale; softmax with
// running maximum and sum in float32; out = sum(prob * v) / sum.
#include "api.h"
#include "common.cuh"

#define AG_THREADS 128
#define AG_MAX_HD 256

template <typename TQ, typename TC, typename TO>
__global__ void __launch_bounds__(AG_THREADS)
attention_general_kernel(const TQ* __restrict__ q, long long q_stride, const TC* __restrict__ k_cache,
                         const TC* __restrict__ v_cache, const int* __restrict__ page_table, int pt_width,
                         const int* __restrict__ tok_seq, const int* __restrict__ positions, TO* __restrict__ out,
                         long long out_stride, int nh, int nkv, int hd, float scale, int window, int n_pages,
                         int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    k_cache = pdl_fresh(k_cache);
    v_cache = pdl_fresh(v_cache);
    __shared__ float qs[AG_MAX_HD];
    __shared__ float ps[AG_THREADS];
    __shared__ int pages[AG_THREADS / HB_PAGE_TOKENS + 2];
    __shared__ float scratch[33];
    const int t = blockIdx.x, j = blockIdx.y, tid = threadIdx.x;
    const int g = j / (nh / nkv);
    const int p = positions[t];
    const int* pt = page_table + (size_t)tok_seq[t] * pt_width;
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const TQ* qr = q + (size_t)t * q_stride + (size_t)j * hd;
    for (int d = tid; d < hd; d += AG_THREADS) qs[d] = to_f32(qr[d]);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[AG_MAX_HD / AG_THREADS];
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / AG_THREADS; i++) acc[i] = 0.0f;

    // tiles start on a multiple of the tile size so that a tile touches at most 3 pages
    for (int s0 = (lo / AG_THREADS) * AG_THREADS; s0 <= p; s0 += AG_THREADS) {
        const int first_page = s0 / HB_PAGE_TOKENS;
        if (tid < AG_THREADS / HB_PAGE_TOKENS + 1) {
            const int pg = first_page + tid;
            int page = (pg < pt_width) ? pt[pg] : -1;
            if (page >= n_pages) page = -1;                     // never read outside the cache
            pages[tid] = page;
        }
        __syncthreads();
        const int s = s0 + tid;
        const bool valid = s >= lo && s <= p;
        float sc = -INFINITY;
        if (valid) {
            const int page = pages[s / HB_PAGE_TOKENS - first_page];
            // a key this query sees on a page the table does not hold: a fault of the host's bookkeeping
            if (page < 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            if (page >= 0) {
                const TC* kr = k_cache + cache_offset(page, g, s, nkv, hd);
                float dot = 0.0f;
                for (int d = 0; d < hd; d++) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                sc = dot * scale;
            }
        }
        const float tmax = block_max(sc, scratch);
        const float m_new = fmaxf(m, tmax);
        const float pr = (sc == -INFINITY) ? 0.0f : expf(sc - m_new);
        ps[tid] = pr;
        const float tsum = block_sum(pr, scratch);  // also orders the writes of ps before the reads below
        const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
        l = l * corr + tsum;
        const int n_in_tile = min(AG_THREADS, p - s0 + 1);
#pragma unroll
        for (int i = 0; i < AG_MAX_HD / AG_THREADS; i++) {
            const int d = tid + i * AG_THREADS;
            if (d < hd) {
                float a = acc[i] * corr;
                for (int e = 0; e < n_in_tile; e++) {
                    const float pe = ps[e];
                    if (pe != 0.0f) {
                        const int se = s0 + e;
                        const int page = pages[se / HB_PAGE_TOKENS - first_page];
                        a = fmaf(pe, to_f32(v_cache[cache_offset(page, g, se, nkv, hd) + d]), a);
                    }
                }
                acc[i] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    TO* o = out + (size_t)t * out_stride + (size_t)j * hd;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int i = 0; i < AG_MAX_HD / AG_THREADS; i++) {
        const int d = tid + i * AG_THREADS;
        if (d < hd) o[d] = from_f32<TO>(acc[i] * inv);
    }
}

extern "C" int hb_attention_general(const void* q, int q_dtype, long long q_stride, const void* k_cache,
                                    const void* v_cache, int cache_dtype, const int* page_table, int pt_width,
                                    const int* tok_seq, const int* positions, void* out, int out_dtype,
                                    long long out_stride, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                    float scale, int window, int n_pages, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0 && n_pages > 0, "attention: bad sizes");
    HB_REQUIRE(n_heads % n_kv_heads == 0, "attention: %d heads are no multiple of %d kv heads", n_heads, n_kv_heads);
    HB_REQUIRE(head_dim <= AG_MAX_HD, "attention: head size %d is larger than %d", head_dim, AG_MAX_HD);
    HB_REQUIRE(n_heads <= 65535, "attention: too many heads");
    dim3 grid(n_tokens, n_heads);
    cudaStream_t s = (cudaStream_t)stream;
#define HB_AG_LAUNCH(TQ, TC, TO)                                                                                      \
    hb_launch(attention_general_kernel<TQ, TC, TO>, dim3(grid), dim3(AG_THREADS), 0, s,                                                  \
        (const TQ*)q, q_stride, (const TC*)k_cache, (const TC*)v_cache, page_table, pt_width, tok_seq, positions,     \
        (TO*)out, out_stride, n_heads, n_kv_heads, head_dim, scale, window, n_pages, status)
    if (q_dtype == HB_F32 && cache_dtype == HB_F32 && out_dtype == HB_F32) HB_AG_LAUNCH(float, float, float);
    else if (q_dtype == HB_BF16 && cache_dtype == HB_BF16 && out_dtype == HB_BF16) HB_AG_LAUNCH(bf16, bf16, bf16);
    else return hb_fail("attention: unsupported dtypes q %d cache %d out %d", q_dtype, cache_dtype, out_dtype);
#undef HB_AG_LAUNCH
    return hb_check_launch("attention_general");
}
