// Prefill attention over the paged bfloat16 cache: flash-style, causal, grouped-query, for
// batches of sequences with unequal numbers of new tokens (no padding).
//
// One CTA = 64 consecutive new tokens of one sequence x one query head; each of its 4 warps
// owns 16 query rows.  The keys (already in the cache, this step's included) are walked page
// by page (64 keys) through a cp.async pipeline; scores and the running maximum and sum are
// float32, probabilities are rounded to bfloat16 for the second product, the output is
// normalised at the end.  Query row at position p sees keys max(0, p - window + 1) .. p.
// Formula: cleanroom-transformer/src/cpu_backend.c:102-124; the reference's kernel handles
// one query per warp without tensor cores (cuda_backend.cu:254-306).
//
// Sizes: head size 64 or 128; any head and group counts; anything else is the general kernel's.
#include "api.h"
#include "mma.cuh"

#define AP_THREADS 128
#define AP_ROWS 64
#define AP_STAGES 2
#define AP_LOG2E 1.4426950408889634f

template <int HD>
__global__ void __launch_bounds__(AP_THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                    const int* __restrict__ page_table, int pt_width, const int* __restrict__ seq_start,
                    const int* __restrict__ seq_pos0, bf16* __restrict__ out, long long out_stride, int n_seqs, int nh,
                    int nkv, float scale_log2e, int window, int n_pages, int* status) {
    pdl_trigger();
    pdl_wait();
    q = pdl_fresh(q);
    kc = pdl_fresh(kc);
    vc = pdl_fresh(vc);
    constexpr int ROW_BYTES = HD * 2;
    constexpr int TILE_BYTES = HB_PAGE_TOKENS * ROW_BYTES;
    constexpr int CHUNKS = ROW_BYTES / 16;
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int head = blockIdx.x, g = head / (nh / nkv);

    // which sequence and which block of its new tokens this CTA serves.  Blocks are taken
    // from the back and the heads are the fast grid index: the query blocks that see the most
    // keys start first, for all heads
    int b = 0, blk = gridDim.y - 1 - blockIdx.y;
    for (; b < n_seqs; b++) {
        const int nb = (seq_start[b + 1] - seq_start[b] + AP_ROWS - 1) / AP_ROWS;
        if (blk < nb) break;
        blk -= nb;
    }
    if (b >= n_seqs) return;
    const int t_begin = seq_start[b], n_new = seq_start[b + 1] - t_begin, pos0 = seq_pos0[b];
    const int row_base = blk * AP_ROWS;                       // first new-token index of the CTA
    const int rows_here = min(AP_ROWS, n_new - row_base);
    const int* pt = page_table + (size_t)b * pt_width;

    // this thread's two query rows (index among the sequence's new tokens) and their positions
    const int r0 = row_base + warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int p0 = pos0 + r0, p1 = pos0 + r1;
    const bool v0 = r0 < n_new, v1 = r1 < n_new;
    uint32_t qf[KSTEPS][4];
    {
        const int c = (lane & 3) * 2;
        const bf16* q0 = q + (size_t)(t_begin + r0) * q_stride + (size_t)head * HD;
        const bf16* q1 = q + (size_t)(t_begin + r1) * q_stride + (size_t)head * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c) : 0u;
            qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c) : 0u;
            qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + c + 8) : 0u;
            qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + c + 8) : 0u;
        }
    }
    // key range of the CTA: from the oldest key its first row sees to its last row's own key
    const int first_pos = pos0 + row_base, last_pos = pos0 + row_base + rows_here - 1;
    const int lo_cta = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int p_begin = lo_cta / HB_PAGE_TOKENS, p_end = last_pos / HB_PAGE_TOKENS + 1;
    const int lo0 = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
    const int lo1 = (window > 0 && p1 - window + 1 > 0) ? p1 - window + 1 : 0;
    // this warp's rows span positions [w_first, w_last]
    const int w_first = pos0 + row_base + warp * 16, w_last = w_first + 15;
    const int w_lo = (window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0;

    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    bool bad_page = false;
    auto load_page = [&](int stage, int page_idx) {
        if (page_idx < p_end) {
            // every page of [p_begin, p_end) holds a key that a row of this CTA sees: one that is
            // missing or outside the cache is a fault of the host's bookkeeping
            int page = page_idx < pt_width ? pt[page_idx] : -1;
            if (page < 0 || page >= n_pages) {
                bad_page = true;                                // noted once, behind the loop
                page = 0;                                       // never read outside the cache
            }
            const uint8_t* ksrc = (const uint8_t*)(kc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint8_t* vsrc = (const uint8_t*)(vc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint32_t kdst = smem_base + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
#pragma unroll
            for (int i = tid; i < HB_PAGE_TOKENS * CHUNKS; i += AP_THREADS) {
                const int row = i / CHUNKS, ch = i % CHUNKS;
                const uint32_t off = swizzled<ROW_BYTES>(row, ch);
                cp_async_16(kdst + off, ksrc + (size_t)i * 16);
                cp_async_16(vdst + off, vsrc + (size_t)i * 16);
            }
        }
        cp_async_commit();
    };

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

#pragma unroll
    for (int s = 0; s < AP_STAGES - 1; s++) load_page(s, p_begin + s);

    for (int pi = p_begin; pi < p_end; pi++) {
        const int it = pi - p_begin;
        cp_async_wait<AP_STAGES - 2>();
        __syncthreads();
        load_page((it + AP_STAGES - 1) % AP_STAGES, pi + AP_STAGES - 1);
        const int page_first = pi * HB_PAGE_TOKENS, page_last = page_first + HB_PAGE_TOKENS - 1;
        if (page_first > w_last || page_last < w_lo) continue;          // nothing for this warp's rows here
        const uint32_t kt = smem_base + (it % AP_STAGES) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
            for (int kq = 0; kq < 4; kq++) {                            // 16 keys per ldmatrix
                uint32_t kf[4];
                const int key_row = kq * 16 + ((lane >> 4) << 3) + (lane & 7);
                ldmatrix_x4(kf, kt + swizzled<ROW_BYTES>(key_row, 2 * ks + ((lane >> 3) & 1)));
                mma_bf16_16816(s[2 * kq], qf[ks], kf[0], kf[1]);
                mma_bf16_16816(s[2 * kq + 1], qf[ks], kf[2], kf[3]);
            }
        }
        const bool edge = page_last > w_first || page_first < ((window > 0) ? w_last - window + 1 : 0);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float v = s[nt][e] * scale_log2e;
                if (edge) {
                    const int key = page_first + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pp = (e >> 1) ? p1 : p0, ll = (e >> 1) ? lo1 : lo0;
                    if (key > pp || key < ll) v = -INFINITY;
                }
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float r = mx[h];
            r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, 1));
            r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, 2));
            const float m_new = fmaxf(m[h], r);
            const float m_safe = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = exp2f(m[h] - m_safe);
            m[h] = m_new;
            float sum = 0.0f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float p = exp2f(s[nt][2 * h + e] - m_safe);
                    s[nt][2 * h + e] = p;
                    sum += p;
                }
            l[h] = l[h] * corr + sum;
#pragma unroll
            for (int i = 0; i < HD / 8; i++) {
                o[i][2 * h] *= corr;
                o[i][2 * h + 1] *= corr;
            }
        }
#pragma unroll
        for (int kq = 0; kq < 4; kq++) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * kq][0], s[2 * kq][1]);
            pa[1] = pack_bf16(s[2 * kq][2], s[2 * kq][3]);
            pa[2] = pack_bf16(s[2 * kq + 1][0], s[2 * kq + 1][1]);
            pa[3] = pack_bf16(s[2 * kq + 1][2], s[2 * kq + 1][3]);
            const int v_row = kq * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
            for (int dn = 0; dn < HD / 16; dn++) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, vt + swizzled<ROW_BYTES>(v_row, 2 * dn + (lane >> 4)));
                mma_bf16_16816(o[2 * dn], pa, vf[0], vf[1]);
                mma_bf16_16816(o[2 * dn + 1], pa, vf[2], vf[3]);
            }
        }
    }
    cp_async_wait<0>();
    if (bad_page && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);

#pragma unroll
    for (int h = 0; h < 2; h++) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    const float inv0 = l[0] > 0.0f ? 1.0f / l[0] : 0.0f, inv1 = l[1] > 0.0f ? 1.0f / l[1] : 0.0f;
    const int c = (lane & 3) * 2;
    if (v0) {
        bf16* dst = out + (size_t)(t_begin + r0) * out_stride + (size_t)head * HD + c;
#pragma unroll
        for (int i = 0; i < HD / 8; i++) *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
    }
    if (v1) {
        bf16* dst = out + (size_t)(t_begin + r1) * out_stride + (size_t)head * HD + c;
#pragma unroll
        for (int i = 0; i < HD / 8; i++) *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

extern "C" int hb_attention_prefill_supported(int n_heads, int n_kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && n_kv_heads > 0 && n_heads % n_kv_heads == 0;
}

template <int HD>
static int launch_prefill(const void* q, long long q_stride, const void* kc, const void* vc, const int* page_table,
                          int pt_width, const int* seq_start, const int* seq_pos0, void* out, long long out_stride,
                          int n_seqs, int q_blocks, int nh, int nkv, float scale, int window, int n_pages, int* status,
                          cudaStream_t s) {
    constexpr int SMEM = AP_STAGES * 2 * HB_PAGE_TOKENS * HD * 2;
    static bool attr_done[HB_MAX_DEVICES] = {};
    bool& attr_set = attr_done[hb_device_slot()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_prefill: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid(nh, q_blocks);
    hb_launch(attn_prefill_kernel<HD>, dim3(grid), dim3(AP_THREADS), SMEM, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, page_table,
                                                           pt_width, seq_start, seq_pos0, (bf16*)out, out_stride, n_seqs, nh, nkv,
                                                           scale * AP_LOG2E, window, n_pages, status);
    return hb_check_launch("attention_prefill");
}

// q: [tokens, q_stride] bfloat16 (head j at columns [j*hd, (j+1)*hd)); seq_start[n_seqs + 1]
// are the token offsets of the sequences, seq_pos0[n_seqs] their lengths before this step;
// q_blocks = sum over sequences of ceil(new tokens / 64).
extern "C" int hb_attention_prefill(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                    const int* page_table, int pt_width, const int* seq_start, const int* seq_pos0,
                                    void* out, long long out_stride, int n_seqs, int q_blocks, int n_heads, int n_kv_heads,
                                    int head_dim, float scale, int window, int n_pages, int* status, void* stream) {
    if (n_seqs == 0 || q_blocks == 0) return 0;
    HB_REQUIRE(hb_attention_prefill_supported(n_heads, n_kv_heads, head_dim),
               "attention_prefill: head size %d with %d heads over %d kv heads is not built (64 or 128)", head_dim, n_heads,
               n_kv_heads);
    HB_REQUIRE(n_seqs > 0 && q_blocks > 0 && q_blocks <= 65535, "attention_prefill: bad sizes");
    HB_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0,
               "attention_prefill: queries and output must be 4-byte aligned");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_prefill: cache must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        return launch_prefill<128>(q, q_stride, k_cache, v_cache, page_table, pt_width, seq_start, seq_pos0, out, out_stride,
                                   n_seqs, q_blocks, n_heads, n_kv_heads, scale, window, n_pages, status, s);
    return launch_prefill<64>(q, q_stride, k_cache, v_cache, page_table, pt_width, seq_start, seq_pos0, out, out_stride, n_seqs,
                              q_blocks, n_heads, n_kv_heads, scale, window, n_pages, status, s);
}
