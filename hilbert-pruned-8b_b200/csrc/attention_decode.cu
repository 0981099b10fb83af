// Decode attention over the paged bfloat16 cache: one query token per sequence, the keys
// split over several CTAs (split-K), partial results combined by a second kernel.
//
// Per (sequence, kv head, split): the CTA streams its pages of keys and values once through a
// 3-stage cp.async pipeline and serves all query heads of the group at once (the group's
// heads are the rows of a 16-row mma.sync tile), so a key is read once per kv head, not once
// per query head.  Scores, running maximum and sum are float32; the split's unnormalised
// output with its maximum and sum goes to scratch; the combine kernel merges the splits with
// log-sum-exp weights and writes bfloat16.  Formula: cleanroom-transformer/src/cpu_backend.c:102-124
// (the reference's GPU kernel reads every key once per query head: cuda_backend.cu:254-306).
//
// Sizes: head size 64 or 128, group size up to 16; anything else is the general kernel's.
#include "api.h"
#include "mma.cuh"

#define AD_THREADS 128
#define AD_STAGES 3
#define AD_LOG2E 1.4426950408889634f
#define AD_MAX_SPLITS 16         // the one-launch kernel keeps (maximum, sum) of every split of a group in shared memory

// The work of one CTA on its range of pages [p_begin, p_end): scores, online softmax and
// weighted values of the group's query heads (fragments `qf`, rows >= group size zero), each of
// the 4 warps on a quarter of every page.  Leaves per-warp results in shared memory:
// so[4][16][HD] unnormalised outputs, sm[4][16] maxima (log2 domain), sl[4][16] sums.
// `after_prologue` runs once the first pages are requested and before any of them is used: the
// place to build the query fragments (and to append a new key) while the loads are in flight.
// `fresh_page` (>= 0): the logical page the kernel in front writes to; the pages before it are
// requested BEFORE griddepcontrol.wait (they hold older tokens only, and the page table and
// the positions come from a copy that finished before the step's first kernel), the wait
// happens before the first request of that page, or after the prologue.  -1: the caller
// has waited already.  `after_wait` runs right after the wait (the place to write that page).
// `status`, `batch_row`: where a page number outside the cache is noted (common.cuh).
// `patch_page` (>= 0): when that page has arrived, row `patch_row` of its key and value tiles is
// overwritten with k_new / v_new (HD values each, in shared memory): the new token's key and
// value, for a page that was requested before they existed.
template <int HD, int STAGES, typename F, typename W>
__device__ __forceinline__ void decode_split_core(uint32_t (&qf)[HD / 16][4], const bf16* kc, const bf16* vc,
                                                  const int* __restrict__ pt, int n_pages, int nkv, int g, int lo,
                                                  int len, int p_begin, int p_end, float scale_log2e, uint8_t* smem,
                                                  F&& after_prologue, int fresh_page, W&& after_wait, int patch_page = -1,
                                                  int patch_row = 0, const bf16* k_new = nullptr, const bf16* v_new = nullptr,
                                                  int* status = nullptr, int batch_row = 0) {
    constexpr int ROW_BYTES = HD * 2;
    constexpr int TILE_BYTES = HB_PAGE_TOKENS * ROW_BYTES;        // one page of K (or V) of one kv head
    constexpr int CHUNKS = ROW_BYTES / 16;
    constexpr int KSTEPS = HD / 16;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem);
    bool bad_page = false;
    auto load_page = [&](int stage, int page_idx) {
        if (page_idx < p_end) {
            // every page of [p_begin, p_end) holds a key the query sees: one that is missing from the
            // table or outside the cache is a fault of the host's bookkeeping (noted, not trapped)
            int page = pt[page_idx];
            if (page < 0 || page >= n_pages) {
                bad_page = true;                            // noted once, behind the loop
                page = 0;                                   // never read outside the cache
            }
            const uint8_t* ksrc = (const uint8_t*)(kc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint8_t* vsrc = (const uint8_t*)(vc + ((size_t)page * nkv + g) * HB_PAGE_TOKENS * HD);
            const uint32_t kdst = smem_base + stage * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
#pragma unroll
            for (int i = tid; i < HB_PAGE_TOKENS * CHUNKS; i += AD_THREADS) {
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

    bool waited = fresh_page < 0;
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (!waited && p_begin + s >= fresh_page) {
            pdl_wait();
            after_wait();
            waited = true;
        }
        load_page(s, p_begin + s);
    }
    if (!waited) {
        pdl_wait();
        after_wait();
    }
    after_prologue();

    for (int pi = p_begin; pi < p_end; pi++) {
        const int it = pi - p_begin;
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        load_page((it + STAGES - 1) % STAGES, pi + STAGES - 1);
        const uint32_t kt = smem_base + (it % STAGES) * 2 * TILE_BYTES, vt = kt + TILE_BYTES;
        if (pi == patch_page) {
            if (tid < 2 * CHUNKS) {
                const int ch = tid % CHUNKS;
                const bool value = tid >= CHUNKS;
                const uint4 x = reinterpret_cast<const uint4*>(value ? v_new : k_new)[ch];
                *reinterpret_cast<uint4*>(smem + (it % STAGES) * 2 * TILE_BYTES + (value ? TILE_BYTES : 0) +
                                          swizzled<ROW_BYTES>(patch_row, ch)) = x;
            }
            __syncthreads();
        }

        // scores of this warp's 16 keys of the page
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
        const int key_row = warp * 16 + ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            uint32_t kf[4];
            ldmatrix_x4(kf, kt + swizzled<ROW_BYTES>(key_row, 2 * ks + ((lane >> 3) & 1)));
            mma_bf16_16816(s[0], qf[ks], kf[0], kf[1]);
            mma_bf16_16816(s[1], qf[ks], kf[2], kf[3]);
        }
        const int key0 = pi * HB_PAGE_TOKENS + warp * 16 + (lane & 3) * 2;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = key0 + nt * 8 + (e & 1);
                const float v = (key >= lo && key < len) ? s[nt][e] * scale_log2e : -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        uint32_t pa[4];
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
            for (int nt = 0; nt < 2; nt++)
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
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        const int v_row = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
        for (int dn = 0; dn < HD / 16; dn++) {
            uint32_t vf[4];
            ldmatrix_x4_trans(vf, vt + swizzled<ROW_BYTES>(v_row, 2 * dn + (lane >> 4)));
            mma_bf16_16816(o[2 * dn], pa, vf[0], vf[1]);
            mma_bf16_16816(o[2 * dn + 1], pa, vf[2], vf[3]);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    if (bad_page && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + batch_row);

    // merge the four warps (each saw a quarter of every page) and write the split's partial
#pragma unroll
    for (int h = 0; h < 2; h++) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    float* so = reinterpret_cast<float*>(smem);                       // [4 warps][16 rows][HD]
    float* sm = so + 4 * 16 * HD;                                      // [4][16]
    float* sl = sm + 4 * 16;
    {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < HD / 8; i++) {
            float* row0 = so + ((size_t)(warp * 16 + r0) * HD) + i * 8 + c;
            float* row1 = row0 + 8 * HD;
            row0[0] = o[i][0];
            row0[1] = o[i][1];
            row1[0] = o[i][2];
            row1[1] = o[i][3];
        }
        if ((lane & 3) == 0) {
            sm[warp * 16 + r0] = m[0];
            sm[warp * 16 + r0 + 8] = m[1];
            sl[warp * 16 + r0] = l[0];
            sl[warp * 16 + r0 + 8] = l[1];
        }
    }
    __syncthreads();
}

// The last split of a (sequence, kv head) to get here combines all of them: a counter per pair
// (left at zero), then the weights of the splits, one (row, split) pair per thread (all maxima
// and sums requested at once), then all partial outputs: two round trips.  Called by every
// thread of the block after it has written its partial result.
template <int HD>
__device__ __forceinline__ void combine_by_last_split(int b, int g, int G, int S, int nh, int nkv, const float* part_o,
                                                      const float* part_ml, int* counters, bf16* out, long long out_stride,
                                                      float* w_split, float* l_split, int* is_last_flag) {
    const int tid = threadIdx.x;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int prev = atomicAdd(counters + (size_t)b * nkv + g, 1);
        const int last = prev == S - 1;
        if (last) counters[(size_t)b * nkv + g] = 0;     // ready for the next launch
        *is_last_flag = last;
    }
    __syncthreads();
    if (!*is_last_flag) return;
    __threadfence();
    for (int i = tid; i < G * S; i += AD_THREADS) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml) + ((size_t)b * nh + g * G) * S + i);
        w_split[i] = ml.x;
        l_split[i] = ml.y;
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY;
        for (int zz = 0; zz < S; zz++) M = fmaxf(M, w_split[tid * S + zz]);
        float L = 0.0f;
        for (int zz = 0; zz < S; zz++) {
            const float mz = w_split[tid * S + zz];
            const float e = mz != -INFINITY ? exp2f(mz - M) : 0.0f;
            L += l_split[tid * S + zz] * e;
            w_split[tid * S + zz] = e;
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        for (int zz = 0; zz < S; zz++) w_split[tid * S + zz] *= inv;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += AD_THREADS) {
        const int r = idx / HD, d = idx - r * HD, head = g * G + r;
        const float* po = part_o + ((size_t)b * nh + head) * S * HD + d;
        float acc = 0.0f;
#pragma unroll 4
        for (int zz = 0; zz < S; zz++) {
            const float w = w_split[r * S + zz];
            const float v = __ldcg(po + (size_t)zz * HD);
            if (w != 0.0f) acc += v * w;
        }
        out[(size_t)b * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc);
    }
}

// The pages [p_begin, p_end) that split z of S takes of a sequence whose keys lo .. len-1 count:
// equal shares of THIS sequence's pages, not of the longest sequence's or of the page table's
// width, so that every split has work whatever the length (a sequence a little above half the
// table's width would leave half the splits empty otherwise).
// `pt_width` bounds the pages: a position beyond the page table reads nothing outside it.
__device__ __forceinline__ void split_pages(int z, int S, int lo, int len, int pt_width, int& p_begin, int& p_end,
                                            int& per_split) {
    const int first = lo / HB_PAGE_TOKENS, last = min((len + HB_PAGE_TOKENS - 1) / HB_PAGE_TOKENS, pt_width);
    per_split = max(1, (last - first + S - 1) / S);
    p_begin = first + z * per_split;
    p_end = min(p_begin + per_split, last);
}

// COMBINE: the last split of a (sequence, kv head) to finish also combines the splits (no
// second kernel); with one split the result goes straight to `out`.
template <int HD, bool COMBINE>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_kernel(const bf16* __restrict__ q, long long q_stride, const bf16* __restrict__ kc, const bf16* __restrict__ vc,
                   const int* __restrict__ page_table, int pt_width, const int* __restrict__ positions,
                   float* part_o, float* part_ml, int nh, int nkv, float scale_log2e,
                   int window, int n_pages, int* counters, bf16* out, long long out_stride, int* status) {
    __shared__ int is_last;
    __shared__ float w_split[COMBINE ? 16 * AD_MAX_SPLITS : 1];
    __shared__ float l_split[COMBINE ? 16 * AD_MAX_SPLITS : 1];
    pdl_trigger();
    // positions and page table come from the step's metadata copy, which finished before the
    // step's first kernel: they may be read before the wait for the kernel in front
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    const int z = blockIdx.x, g = blockIdx.y, b = blockIdx.z, S = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31;
    const int G = nh / nkv;
    const int len = positions[b] + 1;
    const int lo = (window > 0 && len - window > 0) ? len - window : 0;
    int p_begin, p_end, pages_per_split;
    split_pages(z, S, lo, len, pt_width, p_begin, p_end, pages_per_split);
    const int* pt = page_table + (size_t)b * pt_width;

    if (p_begin >= p_end) {                       // nothing to read: an empty partial
        pdl_wait();                               // the scratch may still be read by the step before
        if (tid < G) {
            float* ml = part_ml + (((size_t)b * nh + g * G + tid) * S + z) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.0f;
        }
        if (COMBINE) {
            if (S == 1) {
                for (int idx = tid; idx < G * HD; idx += AD_THREADS)
                    out[(size_t)b * out_stride + (size_t)(g * G) * HD + idx] = __float2bfloat16_rn(0.0f);
            } else {
                combine_by_last_split<HD>(b, g, G, S, nh, nkv, part_o, part_ml, counters, out, out_stride, w_split, l_split, &is_last);
            }
        }
        return;
    }

    // query fragments: row r of the tile is head g*G + r (rows >= G are zero); read after the
    // wait for the kernel in front (which rotated them), while the first pages are in flight.
    // ld.global.cg, not a plain load: the pointer is const __restrict__, and a plain load from
    // it counts as a load from memory that never changes, which the compiler may move above
    // the wait (it did: the queries of the layer before came back).
    uint32_t qf[KSTEPS][4];
    decode_split_core<HD, AD_STAGES>(qf, kc, vc, pt, n_pages, nkv, g, lo, len, p_begin, p_end, scale_log2e, smem, [&] {
        const int r0 = lane >> 2, c = (lane & 3) * 2;
        const unsigned int* q0 = reinterpret_cast<const unsigned int*>(q + (size_t)b * q_stride + (size_t)(g * G + r0) * HD + c);
        const unsigned int* q1 = q0 + 8 * HD / 2;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            qf[ks][0] = r0 < G ? __ldcg(q0 + ks * 8) : 0u;
            qf[ks][1] = r0 + 8 < G ? __ldcg(q1 + ks * 8) : 0u;
            qf[ks][2] = r0 < G ? __ldcg(q0 + ks * 8 + 4) : 0u;
            qf[ks][3] = r0 + 8 < G ? __ldcg(q1 + ks * 8 + 4) : 0u;
        }
    }, (len - 1) / HB_PAGE_TOKENS, [] {}, -1, 0, nullptr, nullptr, status, b);
    if (tid == 0 && len > pt_width * HB_PAGE_TOKENS) hb_note(status, HB_STATUS_PAGE, 1 + b);   // a position beyond the table
    const float* so = reinterpret_cast<const float*>(smem);
    const float* sm = so + 4 * 16 * HD;
    const float* sl = sm + 4 * 16;
    for (int idx = tid; idx < G * HD; idx += AD_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, sm[w * 16 + r]);
        float acc = 0.0f, L = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float e = exp2f(sm[w * 16 + r] - M);
                acc += so[(size_t)(w * 16 + r) * HD + d] * e;
                L += sl[w * 16 + r] * e;
            }
        }
        if (COMBINE && S == 1) {                  // the only split: the result itself
            out[(size_t)b * out_stride + (size_t)(g * G + r) * HD + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
            continue;
        }
        const size_t base = ((size_t)b * nh + g * G + r) * S + z;
        part_o[base * HD + d] = acc;
        if (d == 0) {
            part_ml[base * 2] = M;
            part_ml[base * 2 + 1] = L;
        }
    }
    if (COMBINE && S > 1)
        combine_by_last_split<HD>(b, g, G, S, nh, nkv, part_o, part_ml, counters, out, out_stride, w_split, l_split, &is_last);
}

// The attention of a decode step without a rotation kernel in front: rotate the new token's
// queries and key, append key and value to the cache, attend over the cache in splits.  COMBINE:
// the last split of a (sequence, kv head) to finish combines the partial results (a counter per
// pair, left at zero); else the combination kernel follows.  qkv holds the projections BEFORE
// rotation; it is not written.  All pages of a split are requested before the wait for the
// kernel in front; the split that owns the page of the new position puts the new key and value
// into its copy of that page in shared memory (and into the cache, for the steps to come).
template <int HD, bool COMBINE, int STAGES>
__global__ void __launch_bounds__(AD_THREADS)
attn_decode_fused_kernel(const bf16* __restrict__ qkv, long long qkv_stride, const float2* __restrict__ table, int rot,
                         bf16* kc, bf16* vc, const int* __restrict__ page_table, int pt_width,
                         const int* __restrict__ positions, float* __restrict__ part_o, float* __restrict__ part_ml,
                         int* __restrict__ counters, bf16* __restrict__ out, long long out_stride, int nh, int nkv,
                         float scale_log2e, int window, int n_pages, int append, int* status) {
    pdl_trigger();
    constexpr int KSTEPS = HD / 16;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ int is_last;
    __shared__ __align__(16) bf16 q_rot[16 * HD];          // the group's rotated queries, rows >= G zero
    __shared__ __align__(16) bf16 kv_new[2 * HD];          // the new token's rotated key, then its value
    __shared__ float w_split[COMBINE ? 16 * AD_MAX_SPLITS : 1];   // maxima, then combination weights [row][split]
    __shared__ float l_split[COMBINE ? 16 * AD_MAX_SPLITS : 1];   // sums [row][split]
    const int z = blockIdx.x, g = blockIdx.y, b = blockIdx.z, S = gridDim.x;
    const int tid = threadIdx.x, lane = tid & 31;
    const int G = nh / nkv;
    const int pos = positions[b], len = pos + 1;
    const int lo = (window > 0 && len - window > 0) ? len - window : 0;
    int p_begin, p_end, pages_per_split;
    split_pages(z, S, lo, len, pt_width, p_begin, p_end, pages_per_split);
    const int* pt = page_table + (size_t)b * pt_width;
    // what the kernels in front wrote (projections, table) is read after the wait only, through
    // pointers that the compiler cannot take for memory that never changes
    const bf16* row = nullptr;
    const float2* cs_row = nullptr;
    auto waited = [&]() {
        row = pdl_fresh(qkv) + (size_t)b * qkv_stride;
        cs_row = pdl_fresh(table) + (size_t)b * (rot >> 1);
    };

    // The split that owns the page of the new position rotates the new key and writes it and the
    // value to the cache, for later steps.  This step reads them from shared memory: the page is
    // requested with all the others before the wait, and its row of the new position is
    // overwritten when it has arrived.  The loads are requested together with the queries'.
    const bool owner = append && z == (pos / HB_PAGE_TOKENS - lo / HB_PAGE_TOKENS) / pages_per_split;
    const int half = rot >> 1;
    float kx1 = 0.0f, kx2 = 0.0f;               // one pair of the key per thread (tid < rot/2), or
    float2 kcs = make_float2(1.0f, 0.0f);       // one element beyond the rotated ones (tid >= rot)
    bf16 vx = __float2bfloat16_rn(0.0f);
    auto load_new = [&]() {
        static_assert(HD <= AD_THREADS, "one thread per element of the new key and value");
        const bf16* kn = row + (size_t)(nh + g) * HD;
        const bf16* vn = row + (size_t)(nh + nkv + g) * HD;
        if (tid < half) {
            kcs = cs_row[tid];
            kx1 = __bfloat162float(kn[tid]);
            kx2 = __bfloat162float(kn[tid + half]);
        } else if (tid >= rot && tid < HD) {
            kx1 = __bfloat162float(kn[tid]);
        }
        if (tid < HD) vx = vn[tid];
    };
    auto append_new = [&]() {
        const int page = pos / HB_PAGE_TOKENS < pt_width ? pt[pos / HB_PAGE_TOKENS] : -1;
        const bool in_cache = page >= 0 && page < n_pages;   // the host reserved the page: else a fault of its bookkeeping
        if (!in_cache && tid == 0) hb_note(status, HB_STATUS_PAGE, 1 + b);    // never write outside the cache
        const size_t off = in_cache ? cache_offset(page, g, pos, nkv, HD) : 0;
        if (tid < half) {
            float y1, y2;
            rope_pair(kx1, kx2, kcs.x, kcs.y, y1, y2);
            const bf16 k1 = __float2bfloat16_rn(y1), k2 = __float2bfloat16_rn(y2);
            kv_new[tid] = k1;
            kv_new[tid + half] = k2;
            if (in_cache) {
                kc[off + tid] = k1;
                kc[off + tid + half] = k2;
            }
        } else if (tid >= rot && tid < HD) {
            const bf16 k = __float2bfloat16_rn(kx1);
            kv_new[tid] = k;
            if (in_cache) kc[off + tid] = k;
        }
        if (tid < HD) {
            kv_new[HD + tid] = vx;
            if (in_cache) vc[off + tid] = vx;
        }
    };

    if (p_begin < p_end) {
        uint32_t qf[KSTEPS][4];
        for (int idx = G * HD + tid; idx < 16 * HD; idx += AD_THREADS) q_rot[idx] = __float2bfloat16_rn(0.0f);
        decode_split_core<HD, STAGES>(qf, kc, vc, pt, n_pages, nkv, g, lo, len, p_begin, p_end, scale_log2e, smem, [&]() {
            // the group's queries, rotated once by the whole block; row r of the tile is head
            // g*G + r (rows >= G stay zero), fragments come from shared memory.  One pair
            // (i, i + rot/2) per item.
            const bf16* qrow = row + (size_t)(g * G) * HD;
            constexpr int ITEMS = 16 * (HD / 2) / AD_THREADS;     // G <= 16, rot <= HD
            float x1[ITEMS], x2[ITEMS];
            float2 cs[ITEMS];
#pragma unroll
            for (int u = 0; u < ITEMS; u++) {                     // all loads first: one round trip
                const int idx = tid + u * AD_THREADS;
                if (idx < G * half) {
                    const int r = idx / half, i = idx - r * half;
                    cs[u] = cs_row[i];
                    x1[u] = __bfloat162float(qrow[r * HD + i]);
                    x2[u] = __bfloat162float(qrow[r * HD + i + half]);
                }
            }
            if (owner) {
                load_new();
                append_new();
            }
#pragma unroll
            for (int u = 0; u < ITEMS; u++) {
                const int idx = tid + u * AD_THREADS;
                if (idx < G * half) {
                    const int r = idx / half, i = idx - r * half;
                    float y1, y2;
                    rope_pair(x1[u], x2[u], cs[u].x, cs[u].y, y1, y2);
                    q_rot[r * HD + i] = __float2bfloat16_rn(y1);
                    q_rot[r * HD + i + half] = __float2bfloat16_rn(y2);
                }
            }
            for (int idx = tid; idx < G * (HD - rot); idx += AD_THREADS) {
                const int r = idx / (HD - rot), d = rot + idx - r * (HD - rot);
                q_rot[r * HD + d] = qrow[r * HD + d];
            }
            __syncthreads();
            const int r0 = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                qf[ks][0] = *reinterpret_cast<const uint32_t*>(q_rot + r0 * HD + ks * 16 + c);
                qf[ks][1] = *reinterpret_cast<const uint32_t*>(q_rot + (r0 + 8) * HD + ks * 16 + c);
                qf[ks][2] = *reinterpret_cast<const uint32_t*>(q_rot + r0 * HD + ks * 16 + c + 8);
                qf[ks][3] = *reinterpret_cast<const uint32_t*>(q_rot + (r0 + 8) * HD + ks * 16 + c + 8);
            }
            // Before the wait only pages that no kernel of this step writes may be requested.  A layer
            // that appends writes the new token's row itself (and patches its copy); one that reads
            // another layer's cache finds that row written earlier in this step, so the new token's
            // page is requested after the wait.
        }, append ? (1 << 30) : pos / HB_PAGE_TOKENS, waited, owner ? pos / HB_PAGE_TOKENS : -1, pos % HB_PAGE_TOKENS, kv_new,
           kv_new + HD, status, b);
        const float* so = reinterpret_cast<const float*>(smem);
        const float* sm = so + 4 * 16 * HD;
        const float* sl = sm + 4 * 16;
        for (int idx = tid; idx < G * HD; idx += AD_THREADS) {
            const int r = idx / HD, d = idx - r * HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; w++) M = fmaxf(M, sm[w * 16 + r]);
            float acc = 0.0f, L = 0.0f;
            if (M != -INFINITY) {
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const float e = exp2f(sm[w * 16 + r] - M);
                    acc += so[(size_t)(w * 16 + r) * HD + d] * e;
                    L += sl[w * 16 + r] * e;
                }
            }
            if (COMBINE && S == 1) {                 // the only split: the result itself
                out[(size_t)b * out_stride + (size_t)(g * G + r) * HD + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
                continue;
            }
            const size_t base = ((size_t)b * nh + g * G + r) * S + z;
            part_o[base * HD + d] = acc;
            if (d == 0) {
                part_ml[base * 2] = M;
                part_ml[base * 2 + 1] = L;
            }
        }
    } else {                                     // nothing to read: an empty partial
        pdl_wait();                              // the scratch may still be read by the kernels in front
        waited();
        if (owner) {
            load_new();
            append_new();
        }
        if (tid < G) {
            float* ml = part_ml + (((size_t)b * nh + g * G + tid) * S + z) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.0f;
        }
        if (COMBINE && S == 1)
            for (int idx = tid; idx < G * HD; idx += AD_THREADS)
                out[(size_t)b * out_stride + (size_t)(g * G) * HD + idx] = __float2bfloat16_rn(0.0f);
    }

    if (COMBINE && S > 1)
        combine_by_last_split<HD>(b, g, G, S, nh, nkv, part_o, part_ml, counters, out, out_stride, w_split, l_split, &is_last);
}

// out[b, head, :] = sum_z o_z 2^(m_z - M) / sum_z l_z 2^(m_z - M)
template <typename TO>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           TO* __restrict__ out, long long out_stride, int nh, int hd, int S) {
    pdl_trigger();
    pdl_wait();
    part_o = pdl_fresh(part_o);
    part_ml = pdl_fresh(part_ml);
    const int b = blockIdx.x, head = blockIdx.y;
    const size_t base = ((size_t)b * nh + head) * S;
    float M = -INFINITY;
    for (int z = 0; z < S; z++) M = fmaxf(M, part_ml[(base + z) * 2]);
    float L = 0.0f;
    for (int z = 0; z < S; z++) {
        const float mz = part_ml[(base + z) * 2];
        if (mz != -INFINITY) L += part_ml[(base + z) * 2 + 1] * exp2f(mz - M);
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.0f;
        for (int z = 0; z < S; z++) {
            const float mz = part_ml[(base + z) * 2];
            if (mz != -INFINITY) acc += part_o[(base + z) * hd + d] * exp2f(mz - M);
        }
        out[(size_t)b * out_stride + (size_t)head * hd + d] = from_f32<TO>(acc * inv);
    }
}

extern "C" int hb_attention_decode_supported(int n_heads, int n_kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && n_kv_heads > 0 && n_heads % n_kv_heads == 0 &&
           n_heads / n_kv_heads <= 16;
}

// Scratch floats a call needs: partial outputs and (max, sum) pairs.
extern "C" long long hb_attention_decode_scratch_floats(int batch, int n_heads, int head_dim, int splits) {
    return (long long)batch * n_heads * splits * (head_dim + 2);
}

// counters == nullptr: the splits are combined by a second kernel.
template <int HD, bool COMBINE>
static int launch_decode_splits(const void* q, long long q_stride, const void* kc, const void* vc, const int* page_table,
                                int pt_width, const int* positions, float* part_o, float* part_ml, int* counters, void* out,
                                long long out_stride, int batch, int nh, int nkv, float scale, int window, int splits,
                                int n_pages, int* status, cudaStream_t s) {
    constexpr int PIPE = AD_STAGES * 2 * HB_PAGE_TOKENS * HD * 2;
    constexpr int MERGE = (4 * 16 * HD + 2 * 4 * 16) * 4;
    constexpr int SMEM = PIPE > MERGE ? PIPE : MERGE;
    static bool attr_done[HB_MAX_DEVICES] = {};
    bool& attr_set = attr_done[hb_device_slot()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, COMBINE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_decode: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    hb_launch(attn_decode_kernel<HD, COMBINE>, dim3(splits, nkv, batch), dim3(AD_THREADS), SMEM, s, (const bf16*)q, q_stride,
              (const bf16*)kc, (const bf16*)vc, page_table, pt_width, positions, part_o, part_ml, nh, nkv, scale * AD_LOG2E, window,
              n_pages, counters, (bf16*)out, out_stride, status);
    return hb_check_launch("attention_decode");
}

template <int HD>
static int launch_decode(const void* q, long long q_stride, const void* kc, const void* vc, const int* page_table,
                         int pt_width, const int* positions, float* scratch, int* counters, void* out, long long out_stride,
                         int batch, int nh, int nkv, float scale, int window, int splits, int n_pages,
                         int* status, cudaStream_t s) {
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)batch * nh * splits * HD;
    if (counters != nullptr)
        return launch_decode_splits<HD, true>(q, q_stride, kc, vc, page_table, pt_width, positions, part_o, part_ml, counters, out,
                                              out_stride, batch, nh, nkv, scale, window, splits, n_pages, status, s);
    if (launch_decode_splits<HD, false>(q, q_stride, kc, vc, page_table, pt_width, positions, part_o, part_ml, nullptr, out,
                                        out_stride, batch, nh, nkv, scale, window, splits, n_pages, status, s))
        return 1;
    dim3 cgrid(batch, nh);
    hb_launch(attn_decode_combine_kernel<bf16>, dim3(cgrid), dim3(HD), 0, s, part_o, part_ml, (bf16*)out, out_stride, nh, HD, splits);
    return hb_check_launch("attention_decode_combine");
}

// q: [batch, q_stride] bfloat16 with head j at columns [j*hd, (j+1)*hd); positions[b] is the
// query's position (its own key, already in the cache, is the last one it sees).  `scratch`
// holds hb_attention_decode_scratch_floats floats.  `max_pages` bounds the pages of any
// sequence of the batch; the keys are cut into `splits` ranges of whole pages.
static int attention_decode_any(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                const int* page_table, int pt_width, const int* positions, float* scratch, int* counters,
                                void* out, long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                float scale, int window, int splits, int max_pages, int n_pages, int* status,
                                void* stream) {
    if (batch == 0) return 0;
    HB_REQUIRE(hb_attention_decode_supported(n_heads, n_kv_heads, head_dim),
               "attention_decode: head size %d with %d heads over %d kv heads is not built (64 or 128, groups up to 16)",
               head_dim, n_heads, n_kv_heads);
    HB_REQUIRE(batch > 0 && splits >= 1 && max_pages >= 1 && scratch != nullptr, "attention_decode: bad sizes");
    HB_REQUIRE(pt_width >= 1 && max_pages <= pt_width, "attention_decode: %d pages per sequence do not fit a page table of width %d",
               max_pages, pt_width);
    HB_REQUIRE(batch <= 65535 && n_kv_heads <= 65535, "attention_decode: batch or kv heads too large for one launch");
    HB_REQUIRE(q_stride % 2 == 0 && ((uintptr_t)q & 3) == 0, "attention_decode: queries must be 4-byte aligned");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_decode: cache must be 16-byte aligned");
    if (splits > max_pages) splits = max_pages;
    HB_REQUIRE(counters == nullptr || splits <= AD_MAX_SPLITS, "attention_decode: at most %d splits when the last one combines, got %d",
               AD_MAX_SPLITS, splits);
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        return launch_decode<128>(q, q_stride, k_cache, v_cache, page_table, pt_width, positions, scratch, counters, out,
                                  out_stride, batch, n_heads, n_kv_heads, scale, window, splits, n_pages, status, s);
    return launch_decode<64>(q, q_stride, k_cache, v_cache, page_table, pt_width, positions, scratch, counters, out, out_stride,
                             batch, n_heads, n_kv_heads, scale, window, splits, n_pages, status, s);
}

extern "C" int hb_attention_decode(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                   const int* page_table, int pt_width, const int* positions, float* scratch, void* out,
                                   long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim, float scale,
                                   int window, int splits, int max_pages, int n_pages, int* status, void* stream) {
    return attention_decode_any(q, q_stride, k_cache, v_cache, page_table, pt_width, positions, scratch, nullptr, out, out_stride,
                                batch, n_heads, n_kv_heads, head_dim, scale, window, splits, max_pages, n_pages, status, stream);
}

// The same in ONE launch: the last split of a (sequence, kv head) to finish combines the
// splits.  `counters`: batch * n_kv_heads ints, zero before the first use (left at zero).
extern "C" int hb_attention_decode_combined(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                            const int* page_table, int pt_width, const int* positions, float* scratch,
                                            int* counters, void* out, long long out_stride, int batch, int n_heads,
                                            int n_kv_heads, int head_dim, float scale, int window, int splits, int max_pages,
                                            int n_pages, int* status, void* stream) {
    HB_REQUIRE(counters != nullptr, "attention_decode_combined: no counters");
    return attention_decode_any(q, q_stride, k_cache, v_cache, page_table, pt_width, positions, scratch, counters, out, out_stride,
                                batch, n_heads, n_kv_heads, head_dim, scale, window, splits, max_pages, n_pages, status, stream);
}

#define AD_DEEP_STAGES 6        // when every CTA has an SM of its own: five pages in flight instead of two

template <int HD, bool COMBINE, int STAGES>
static int launch_decode_fused_stages(const void* qkv, long long stride, const float* table, int rot, void* kc, void* vc,
                                      const int* page_table, int pt_width, const int* positions, float* part_o, float* part_ml,
                                      int* counters, void* out, long long out_stride, int batch, int nh, int nkv, float scale,
                                      int window, int splits, int n_pages, int append, int* status, cudaStream_t s) {
    constexpr int PIPE = STAGES * 2 * HB_PAGE_TOKENS * HD * 2;
    constexpr int MERGE = (4 * 16 * HD + 2 * 4 * 16) * 4;
    constexpr int SMEM = PIPE > MERGE ? PIPE : MERGE;
    static_assert(SMEM + 8 * 1024 <= 227 * 1024, "page pipeline does not fit shared memory");
    static bool attr_done[HB_MAX_DEVICES] = {};
    bool& attr_set = attr_done[hb_device_slot()];
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_fused_kernel<HD, COMBINE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_decode_fused: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    hb_launch(attn_decode_fused_kernel<HD, COMBINE, STAGES>, dim3(splits, nkv, batch), dim3(AD_THREADS), SMEM, s, (const bf16*)qkv, stride,
              (const float2*)table, rot, (bf16*)kc, (bf16*)vc, page_table, pt_width, positions, part_o, part_ml, counters,
              (bf16*)out, out_stride, nh, nkv, scale * AD_LOG2E, window, n_pages, append, status);
    return hb_check_launch("attention_decode_fused");
}

static int decode_sm_count() {
    static int count[HB_MAX_DEVICES] = {};
    int& n = count[hb_device_slot()];
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    }
    return n;
}

// With no more CTAs than SMs (one sequence with a long cache) a CTA cannot share an SM anyway:
// the deep pipeline keeps five pages in flight per CTA instead of two.
template <int HD, bool COMBINE>
static int launch_decode_fused_splits(const void* qkv, long long stride, const float* table, int rot, void* kc, void* vc,
                                      const int* page_table, int pt_width, const int* positions, float* part_o, float* part_ml,
                                      int* counters, void* out, long long out_stride, int batch, int nh, int nkv, float scale,
                                      int window, int splits, int n_pages, int append, int* status, cudaStream_t s) {
    if ((long long)splits * nkv * batch <= decode_sm_count())
        return launch_decode_fused_stages<HD, COMBINE, AD_DEEP_STAGES>(qkv, stride, table, rot, kc, vc, page_table, pt_width, positions,
                                                                       part_o, part_ml, counters, out, out_stride, batch, nh, nkv,
                                                                       scale, window, splits, n_pages, append, status, s);
    return launch_decode_fused_stages<HD, COMBINE, AD_STAGES>(qkv, stride, table, rot, kc, vc, page_table, pt_width, positions, part_o,
                                                              part_ml, counters, out, out_stride, batch, nh, nkv, scale, window,
                                                              splits, n_pages, append, status, s);
}

template <int HD>
static int decode_ctas_per_sm() {
    constexpr int PIPE = AD_STAGES * 2 * HB_PAGE_TOKENS * HD * 2;
    constexpr int MERGE = (4 * 16 * HD + 2 * 4 * 16) * 4;
    constexpr int SMEM = PIPE > MERGE ? PIPE : MERGE;
    if (cudaFuncSetAttribute(attn_decode_fused_kernel<HD, false, AD_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn_decode_fused_kernel<HD, false, AD_STAGES>, AD_THREADS, SMEM) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

// How many CTAs of the split-K decode attention one SM holds at once (0: head size not built or
// the query failed): what the host sizes the number of splits with.
extern "C" int hb_attention_decode_ctas_per_sm(int head_dim) {
    if (head_dim == 128) return decode_ctas_per_sm<128>();
    if (head_dim == 64) return decode_ctas_per_sm<64>();
    return 0;
}

// counters == nullptr: the splits (more than one) are combined by a second kernel.
template <int HD>
static int launch_decode_fused(const void* qkv, long long stride, const float* table, int rot, void* kc, void* vc,
                               const int* page_table, int pt_width, const int* positions, float* scratch, int* counters,
                               void* out, long long out_stride, int batch, int nh, int nkv, float scale, int window,
                               int splits, int n_pages, int append, int* status, cudaStream_t s) {
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)batch * nh * splits * HD;
    if (counters != nullptr || splits == 1)
        return launch_decode_fused_splits<HD, true>(qkv, stride, table, rot, kc, vc, page_table, pt_width, positions, part_o,
                                                    part_ml, counters, out, out_stride, batch, nh, nkv, scale, window, splits,
                                                    n_pages, append, status, s);
    if (launch_decode_fused_splits<HD, false>(qkv, stride, table, rot, kc, vc, page_table, pt_width, positions, part_o, part_ml,
                                              nullptr, out, out_stride, batch, nh, nkv, scale, window, splits,
                                              n_pages, append, status, s))
        return 1;
    hb_launch(attn_decode_combine_kernel<bf16>, dim3(batch, nh), dim3(HD), 0, s, part_o, part_ml, (bf16*)out, out_stride, nh, HD, splits);
    return hb_check_launch("attention_decode_combine");
}

// The attention of a decode step in one launch.  qkv: [batch, stride] bfloat16 rows holding the
// q, k and v projections of each sequence's new token BEFORE rotation (q heads first, then k
// heads, then v heads); `table`: [batch, rot/2] (cos, sin) of the tokens' positions;
// positions[b] is the new token's position.  With `append` the rotated key and the value are
// written to the cache first.  `scratch` as for hb_attention_decode; `counters` holds
// batch * n_kv_heads ints, zero before the first use (the kernel leaves them zero), or is
// null: then a second kernel combines the splits.
extern "C" int hb_attention_decode_fused(const void* qkv, long long stride, const float* table, int rot, void* k_cache,
                                         void* v_cache, const int* page_table, int pt_width, const int* positions,
                                         float* scratch, int* counters, void* out, long long out_stride, int batch,
                                         int n_heads, int n_kv_heads, int head_dim, float scale, int window, int splits,
                                         int max_pages, int n_pages, int append, int* status, void* stream) {
    if (batch == 0) return 0;
    HB_REQUIRE(hb_attention_decode_supported(n_heads, n_kv_heads, head_dim),
               "attention_decode_fused: head size %d with %d heads over %d kv heads is not built (64 or 128, groups up to 16)",
               head_dim, n_heads, n_kv_heads);
    HB_REQUIRE(batch > 0 && splits >= 1 && max_pages >= 1 && scratch, "attention_decode_fused: bad sizes");
    HB_REQUIRE(pt_width >= 1 && max_pages <= pt_width, "attention_decode_fused: %d pages per sequence do not fit a page table of width %d",
               max_pages, pt_width);
    HB_REQUIRE(counters == nullptr || splits <= AD_MAX_SPLITS, "attention_decode_fused: at most %d splits when the last one combines, got %d",
               AD_MAX_SPLITS, splits);
    HB_REQUIRE(batch <= 65535 && n_kv_heads <= 65535, "attention_decode_fused: batch or kv heads too large for one launch");
    HB_REQUIRE(rot >= 0 && rot <= head_dim && rot % 2 == 0 && (rot == 0 || table), "attention_decode_fused: bad rotary size %d", rot);
    HB_REQUIRE(stride % 2 == 0 && ((uintptr_t)qkv & 3) == 0, "attention_decode_fused: projections must be 4-byte aligned");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_decode_fused: cache must be 16-byte aligned");
    if (splits > max_pages) splits = max_pages;
    cudaStream_t s = (cudaStream_t)stream;
    if (head_dim == 128)
        return launch_decode_fused<128>(qkv, stride, table, rot, k_cache, v_cache, page_table, pt_width, positions, scratch,
                                        counters, out, out_stride, batch, n_heads, n_kv_heads, scale, window, splits,
                                        n_pages, append, status, s);
    return launch_decode_fused<64>(qkv, stride, table, rot, k_cache, v_cache, page_table, pt_width, positions, scratch,
                                   counters, out, out_stride, batch, n_heads, n_kv_heads, scale, window, splits, n_pages,
                                   append, status, s);
}

// ------------------------------------------------------------------ no-allocation entry point
// See noalloc.h.  The scratch of the split-K kernels is this file-scope device array.  In
// host code the array's name is only a handle: its device address comes from
// cudaGetSymbolAddress, looked up once per device with that device current.
#include <mutex>

#include "noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[HB_NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_address[64];
static std::mutex g_noalloc_mutex;

static int noalloc_scratch_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return hb_fail("attention_decode_noalloc: no current device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return hb_fail("attention_decode_noalloc: device index %d is not supported", dev);
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_address[dev] == nullptr) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return hb_fail("attention_decode_noalloc: cannot find the scratch array on device %d: %s", dev,
                           cudaGetErrorString(e));
        g_noalloc_address[dev] = p;
    }
    *out = g_noalloc_address[dev];
    return 0;
}

extern "C" int hb_attention_decode_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                           const int* page_table, int pt_width, const int* positions, void* out,
                                           long long out_stride, int batch, int n_heads, int n_kv_heads, int head_dim,
                                           float scale, int window, int splits, int max_pages, int n_pages,
                                           void* stream) {
    if (batch == 0) return 0;
    HB_REQUIRE(batch > 0 && splits >= 1 && max_pages >= 1 && n_heads > 0, "attention_decode_noalloc: bad sizes");
    const int used_splits = splits > max_pages ? max_pages : splits;
    const long long need = hb_attention_decode_scratch_floats(batch, n_heads, head_dim, used_splits);
    HB_REQUIRE(need <= (long long)HB_NOALLOC_SCRATCH_FLOATS,
               "attention_decode_noalloc: batch %d x %d heads x %d splits needs %lld scratch floats, the built-in area "
               "holds %d; lower the batch or the splits, or use hb_attention_decode with scratch of your own",
               batch, n_heads, used_splits, need, (int)HB_NOALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (noalloc_scratch_address(&scratch)) return 1;
    return hb_attention_decode(q, q_stride, k_cache, v_cache, page_table, pt_width, positions, scratch, out, out_stride,
                               batch, n_heads, n_kv_heads, head_dim, scale, window, splits, max_pages, n_pages, nullptr, stream);
}
