// Prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head size 64 or 128:
// flash-style, causal, grouped-query, over the paged bfloat16 cache, for batches of sequences
// with unequal numbers of new tokens.
//
// One CTA = 128 consecutive new tokens of one sequence x one query head.  The 128 query rows
// are the 128 lanes of tensor memory.  Keys and values come in tiles of 128 keys (two pages).
//   warp 0     TMA producer: the query tile once, then K tiles and V tiles (three stages of
//              128 keys x head size each, freed separately: a K tile right after S_j, a V tile
//              after O += P_j V_j)
//   warp 1     owns tensor memory; one thread issues the MMAs:
//                S_j = Q K_j^T      (operands in shared memory, K-major, head size / 16 steps)
//                O  += P_j V_j      (P_j from tensor memory, V_j in shared memory as stored:
//                                    keys are rows, an MN-major B operand)
//   warps 2-9  softmax: two threads per query row (64 key columns each): they read S_j from
//              tensor memory, agree on the row's maximum through shared memory, keep the
//              running maximum and sum in float32 and write P_j (bfloat16) over S_j
// Two S buffers: the softmax of tile j runs while the tensor cores compute S_{j+1}.  The
// output accumulator stays in tensor memory; it is rescaled only when a row's maximum grows by
// more than 2^8 (probabilities are taken against a maximum that may be stale by less).
// Formula: cleanroom-transformer/src/cpu_backend.c:102-124 (scores q.k/sqrt(hd) over keys
// lo..p, softmax, weighted values).
//
// Every wait is bounded; a wait that runs out sets *error_flag and the CTA drains and leaves.
#include "api.h"
#include "tcgen05.cuh"

#define FA_ROWS 128
#define FA_KEYS 128
#define FA_HALF_BYTES (128 * 64 * 2)                 // 128 rows x 64 elements: one swizzle-wide sub-tile
#define FA_TILE_BYTES(HD) ((HD) / 64 * FA_HALF_BYTES) // 128 rows x head size, bf16
#define FA_STAGES 3
#define FA_LOG2E 1.4426950408889634f
#define FA_RESCALE_THRESHOLD 8.0f
#define FA_THREADS 320                                // producer, MMA, 8 softmax warps

__device__ __forceinline__ void tmem_ld32(uint32_t addr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(addr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive columns of this thread's lane, loaded and waited for in ONE asm statement, so
// that no use of the values can be scheduled before the wait
__device__ __forceinline__ void tmem_ld64(uint32_t addr, float* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31]), "=f"(v[32]), "=f"(v[33]), "=f"(v[34]), "=f"(v[35]), "=f"(v[36]), "=f"(v[37]), "=f"(v[38]), "=f"(v[39]), "=f"(v[40]), "=f"(v[41]), "=f"(v[42]), "=f"(v[43]), "=f"(v[44]), "=f"(v[45]), "=f"(v[46]), "=f"(v[47]), "=f"(v[48]), "=f"(v[49]), "=f"(v[50]), "=f"(v[51]), "=f"(v[52]), "=f"(v[53]), "=f"(v[54]), "=f"(v[55]), "=f"(v[56]), "=f"(v[57]), "=f"(v[58]), "=f"(v[59]), "=f"(v[60]), "=f"(v[61]), "=f"(v[62]), "=f"(v[63])
        : "r"(addr), "r"(addr + 32)
        : "memory");
}
// 2^x on the special-function unit (float32, about 2 ulp); 2^-inf = 0
__device__ __forceinline__ float exp2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(addr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
}
__device__ __forceinline__ void tmem_st16u(uint32_t addr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16_pair(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A from tensor memory (K-major, bf16 pairs per column), B from shared memory
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory descriptor of an MN-major operand with 128-byte swizzle: rows are K (keys),
// 64 MN elements (128 bytes) per row; 8-row groups `sbo` bytes apart, 64-element MN blocks
// `lbo` bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(sbo >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const int* __restrict__ page_table, int pt_width,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, bf16* __restrict__ out,
                       long long out_stride, int n_seqs, int nh, int nkv, float scale_log2e, int window, int n_pages,
                       int* __restrict__ error_flag) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // [Q tile][K stages 3 x tile][V stages 3 x tile][barriers]; a tile is 128 rows x HD
    constexpr int TILE = FA_TILE_BYTES(HD);
    constexpr int HALVES = HD / 64;                      // swizzle-wide sub-tiles per tile
    uint64_t* bars = (uint64_t*)(smem + TILE + FA_STAGES * 2 * TILE);
    uint32_t* tmem_slot = (uint32_t*)(bars + 18);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* xrow = (float*)(tmem_slot + 4);                    // [2 halves][128 rows]: row maxima, at the end row sums
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t k_smem = smem_base + TILE, v_smem = k_smem + FA_STAGES * TILE;
    const uint32_t q_full = smem_u32(bars), k_full0 = smem_u32(bars + 1), k_empty0 = smem_u32(bars + 4);
    const uint32_t v_full0 = smem_u32(bars + 7), v_empty0 = smem_u32(bars + 10);
    const uint32_t s_full0 = smem_u32(bars + 13), p_full0 = smem_u32(bars + 15), pv_done = smem_u32(bars + 17);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.x, g = head / (nh / nkv);

    // which sequence and which block of its new tokens.  Blocks are taken from the back, and
    // the heads are the fast grid index: the query blocks that see the most keys start first,
    // for all heads, and the short ones fill the gaps at the end (2048 tokens x 32 heads on
    // 148 SMs: 34 block lengths of time instead of 43, ideal 33)
    int b = 0, blk = gridDim.y - 1 - blockIdx.y;
    for (; b < n_seqs; b++) {
        const int nb = (seq_start[b + 1] - seq_start[b] + FA_ROWS - 1) / FA_ROWS;
        if (blk < nb) break;
        blk -= nb;
    }
    const bool has_work = b < n_seqs;
    const int t_begin = has_work ? seq_start[b] : 0, n_new = has_work ? seq_start[b + 1] - t_begin : 0;
    const int pos0 = has_work ? seq_pos0[b] : 0;
    const int row_base = blk * FA_ROWS;
    const int rows_here = min(FA_ROWS, n_new - row_base);
    const int first_pos = pos0 + row_base, last_pos = first_pos + rows_here - 1;
    const int lo_cta = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int jt0 = lo_cta / FA_KEYS, jt1 = has_work ? last_pos / FA_KEYS + 1 : 0;
    const int n_it = jt1 - jt0;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < FA_STAGES; s++) {
            mbar_init(k_full0 + 8 * s, 1);
            mbar_init(k_empty0 + 8 * s, 1);
            mbar_init(v_full0 + 8 * s, 1);
            mbar_init(v_empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(s_full0 + 8 * s, 1);
            mbar_init(p_full0 + 8 * s, 256);
        }
        mbar_init(pv_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_o = tmem_base + 256;               // S buffers at columns 0 and 128, O at 256
    pdl_trigger();
    pdl_wait();                                          // queries, keys and values come from the kernels in front

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && n_it > 0) {
            const int* pt = page_table + (size_t)b * pt_width;
            mbar_expect_tx(q_full, TILE);
            for (int half = 0; half < HALVES; half++)
                tma_load_2d(smem_base + half * FA_HALF_BYTES, &map_q, q_full, head * HD + half * 64, t_begin + row_base);
            // K tiles run ahead of V tiles: a K stage is free as soon as its scores exist
            auto load_tile = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int it) {
                mbar_expect_tx(bar, TILE);
                for (int pg = 0; pg < 2; pg++) {
                    const int pi = (jt0 + it) * 2 + pg;
                    int page = pi < pt_width ? pt[pi] : -1;
                    if (page < 0 || page >= n_pages) {
                        // a tile's second page may lie behind the sequence's end (its keys are masked);
                        // a page between the oldest key the first row sees and the last row's own key
                        // must exist: the host's bookkeeping is at fault.  `error_flag` points at the
                        // status words (common.cuh)
                        if (page >= n_pages || (pi >= lo_cta / HB_PAGE_TOKENS && pi <= last_pos / HB_PAGE_TOKENS))
                            hb_note(error_flag, HB_STATUS_PAGE, 1 + b);
                        page = 0;                                   // never read outside the cache
                    }
                    const int row = (page * nkv + g) * HB_PAGE_TOKENS;
                    for (int half = 0; half < HALVES; half++)
                        tma_load_2d(dst + half * FA_HALF_BYTES + pg * (FA_HALF_BYTES / 2), map, bar, half * 64, row);
                }
            };
            int k_issued = 0, v_issued = 0;
            bool alive = true;
            for (int step = 0; step < n_it + 1 && alive; step++) {
                const int ik = step, iv = step - 1;                 // the K of tile `step`, then the V of the tile before
                if (ik < n_it) {
                    const int s = ik % FA_STAGES;
                    if (!mbar_wait(k_empty0 + 8 * s, ((ik / FA_STAGES) & 1) ^ 1)) {
                        atomicExch(error_flag, 21);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    load_tile(k_smem + s * TILE, &map_k, k_full0 + 8 * s, ik);
                    k_issued = ik + 1;
                }
                if (iv >= 0) {
                    const int s = iv % FA_STAGES;
                    if (!mbar_wait(v_empty0 + 8 * s, ((iv / FA_STAGES) & 1) ^ 1)) {
                        atomicExch(error_flag, 22);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    load_tile(v_smem + s * TILE, &map_v, v_full0 + 8 * s, iv);
                    v_issued = iv + 1;
                }
            }
            for (int it = max(0, k_issued - FA_STAGES); it < k_issued; it++)
                if (!mbar_wait(k_full0 + 8 * (it % FA_STAGES), (it / FA_STAGES) & 1)) atomicExch(error_flag, 23);
            for (int it = max(0, v_issued - FA_STAGES); it < v_issued; it++)
                if (!mbar_wait(v_full0 + 8 * (it % FA_STAGES), (it / FA_STAGES) & 1)) atomicExch(error_flag, 23);
            if (!mbar_wait(q_full, 0)) atomicExch(error_flag, 23);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_qk = instr_desc_bf16_mn(128, FA_KEYS);
            constexpr uint32_t idesc_pv = instr_desc_bf16_mn(128, HD) | (1u << 16);           // B is MN-major
            bool alive = mbar_wait(q_full, 0);
            if (!alive) { atomicExch(error_flag, 24); *abort_flag = 1; }
            auto issue_qk = [&](int it) {
                const int s = it % FA_STAGES, sb = it & 1;
                if (!mbar_wait(k_full0 + 8 * s, (it / FA_STAGES) & 1)) {
                    atomicExch(error_flag, 25);
                    *abort_flag = 1;
                    alive = false;
                    return;
                }
                tc_fence_after();
                const uint32_t kst = k_smem + s * TILE;
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++) {
                    const uint32_t off = (kk >> 2) * FA_HALF_BYTES + (kk & 3) * 32;
                    umma_bf16(tmem_base + sb * 128, smem_desc_sw128(smem_base + off), smem_desc_sw128(kst + off), idesc_qk, kk ? 1u : 0u);
                }
                umma_commit(k_empty0 + 8 * s);                // the K tile is used up
                umma_commit(s_full0 + 8 * sb);
            };
            if (alive) issue_qk(0);
            for (int it = 0; it < n_it && alive; it++) {
                const int s = it & 1;
                if (it + 1 < n_it) issue_qk(it + 1);          // runs while the softmax warps work on tile `it`
                if (!alive) break;
                if (!mbar_wait(p_full0 + 8 * s, (it >> 1) & 1)) {
                    atomicExch(error_flag, 26);
                    *abort_flag = 1;
                    break;
                }
                const int sv = it % FA_STAGES;
                if (!mbar_wait(v_full0 + 8 * sv, (it / FA_STAGES) & 1)) {
                    atomicExch(error_flag, 30);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t vst = v_smem + sv * TILE;
#pragma unroll
                for (int kk = 0; kk < FA_KEYS / 16; kk++)
                    umma_bf16_ts(tm_o, tmem_base + s * 128 + kk * 8, smem_desc_mn_sw128(vst + kk * 16 * 128, FA_HALF_BYTES, 1024),
                                 idesc_pv, (it | kk) ? 1u : 0u);
                umma_commit(v_empty0 + 8 * sv);               // the V tile is used up
                umma_commit(pv_done);
            }
        }
    } else if (n_it > 0) {
        // ---------------------------------------------------------------- softmax and output
        const int q = warp & 3, r = q * 32 + lane;            // query row of this thread = TMEM lane
        const int hf = (warp - 2) >> 2;                       // which 64 key columns (and which half of the output columns) of the row
        constexpr int OC = HD / 2;                            // output columns per thread: 32 or 64
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        const int qpos = first_pos + r;
        const int lo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
        const bool valid = row_base + r < n_new;
        float m_run = -INFINITY, l = 0.0f;                    // l: this thread's columns only
        bool ok = true;
        for (int it = 0; it < n_it; it++) {
            const int s = it & 1;
            if (!mbar_wait(s_full0 + 8 * s, (it >> 1) & 1)) {
                atomicExch(error_flag, 27);
                *abort_flag = 1;
            }
            tc_fence_after();
            const uint32_t tm_s = tmem_base + s * 128 + lane_base;
            const int kbase = (jt0 + it) * FA_KEYS + hf * 64;
            // this thread's row sees keys lo..qpos; as columns of its half tile: [c_lo, c_hi]
            const int c_lo = lo - kbase, c_hi = qpos - kbase;
            // the scores in registers: one round trip to tensor memory
            float sv[64];
            tmem_ld64(tm_s + hf * 64, sv);
            if (c_lo > 0 || c_hi < 63) {                       // the causal diagonal or the window's edge
#pragma unroll
                for (int e = 0; e < 64; e++)
                    if (e < c_lo || e > c_hi) sv[e] = -INFINITY;
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int e = 0; e < 64; e += 4) {
                mx4[0] = fmaxf(mx4[0], sv[e]);
                mx4[1] = fmaxf(mx4[1], sv[e + 1]);
                mx4[2] = fmaxf(mx4[2], sv[e + 2]);
                mx4[3] = fmaxf(mx4[3], sv[e + 3]);
            }
            xrow[hf * 128 + r] = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // all 256 softmax threads: every score is in registers now (P may overwrite S) and the
            // other half's maximum is visible
            asm volatile("bar.sync 2, 256;" ::: "memory");
            if (*abort_flag) {                                 // read after the barrier: the same for all 256 threads
                ok = false;
                break;
            }
            const float m_tile = fmaxf(xrow[r], xrow[128 + r]) * scale_log2e;
            if (it == 0) {
                m_run = m_tile;
            } else {
                const bool grow = m_tile > m_run + FA_RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffu, grow)) {
                    // the accumulator may only be touched between two of its MMAs
                    if (!mbar_wait(pv_done, (it - 1) & 1)) {
                        atomicExch(error_flag, 28);
                        *abort_flag = 1;
                    }
                    tc_fence_after();
                    const float m_new = fmaxf(m_run, m_tile);
                    const float corr = m_new == -INFINITY ? 1.0f : exp2f(m_run - m_new);
                    m_run = m_new;
                    l *= corr;
#pragma unroll 1
                    for (int c = 0; c < OC / 32; c++) {
                        float v[32];
                        tmem_ld32(tm_o + lane_base + hf * OC + c * 32, v);
#pragma unroll
                        for (int e = 0; e < 32; e++) v[e] *= corr;
                        tmem_st32(tm_o + lane_base + hf * OC + c * 32, v);
                    }
                    tmem_wait_st();
                }
            }
            const float neg_m = m_run == -INFINITY ? 0.0f : -m_run;
            float sum2[2] = {0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t pk[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = exp2_approx(fmaf(sv[c * 32 + e], scale_log2e, neg_m));
                    const float p1 = exp2_approx(fmaf(sv[c * 32 + e + 1], scale_log2e, neg_m));
                    sum2[0] += p0;
                    sum2[1] += p1;
                    pk[e >> 1] = pack_bf16_pair(p0, p1);
                }
                tmem_st16u(tm_s + hf * 32 + c * 16, pk);      // P over S
            }
            l += sum2[0] + sum2[1];
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(p_full0 + 8 * s);
        }
        if (ok && !mbar_wait(pv_done, (n_it - 1) & 1)) {
            atomicExch(error_flag, 29);
            *abort_flag = 1;
        }
        // the two halves of a row add their sums
        asm volatile("bar.sync 2, 256;" ::: "memory");      // nobody still reads the maxima
        xrow[hf * 128 + r] = l;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        if (!*abort_flag) {
            tc_fence_after();
            const float lt = xrow[r] + xrow[128 + r];
            const float inv = lt > 0.0f ? 1.0f / lt : 0.0f;
            bf16* dst = out + (size_t)(t_begin + row_base + r) * out_stride + (size_t)head * HD + hf * OC;
#pragma unroll 1
            for (int c = 0; c < OC / 32; c++) {
                float v[32];
                tmem_ld32(tm_o + lane_base + hf * OC + c * 32, v);
                if (valid) {
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        uint4 o4;
                        o4.x = pack_bf16_pair(v[e] * inv, v[e + 1] * inv);
                        o4.y = pack_bf16_pair(v[e + 2] * inv, v[e + 3] * inv);
                        o4.z = pack_bf16_pair(v[e + 4] * inv, v[e + 5] * inv);
                        o4.w = pack_bf16_pair(v[e + 6] * inv, v[e + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + e) = o4;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

extern "C" int hb_attention_prefill_tc_supported(int n_heads, int n_kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && n_kv_heads > 0 && n_heads % n_kv_heads == 0;
}

template <int HD>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const int* page_table, int pt_width,
                             const int* seq_start, const int* seq_pos0, void* out, long long out_stride, int n_seqs, int q_blocks,
                             int n_heads, int n_kv_heads, float scale, int window, int n_pages, int* error_flag, cudaStream_t stream) {
    constexpr int TILE = FA_TILE_BYTES(HD);
    constexpr int SMEM = TILE + FA_STAGES * 2 * TILE + 18 * 8 + 16 + 2 * 128 * 4 + 1024;
    static_assert(SMEM <= 227 * 1024, "attention tiles do not fit shared memory");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("attention_prefill_tc: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    cudaError_t e = hb_launch(attn_prefill_tc_kernel<HD>, dim3(n_heads, q_blocks), dim3(FA_THREADS), SMEM, stream, mq, mk, mv,
                              page_table, pt_width, seq_start, seq_pos0, (bf16*)out, out_stride, n_seqs, n_heads, n_kv_heads,
                              scale * FA_LOG2E, window, n_pages, error_flag);
    if (e != cudaSuccess) return hb_fail("attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
    return hb_check_launch("attention_prefill_tc");
}

// Tensor map over rows of `cols` bfloat16 with row stride `ld`: boxes of 64 columns x box_rows.
// q: [tokens, q_stride] (head j at columns [j*hd, (j+1)*hd)); k_cache / v_cache: one layer,
// [n_pages][n_kv_heads][64][hd]; seq_start / seq_pos0 as for hb_attention_prefill; q_blocks =
// sum over sequences of ceil(new tokens / 128).
extern "C" int hb_attention_prefill_tc(const void* q, long long q_stride, long long n_tokens, const void* k_cache,
                                       const void* v_cache, const int* page_table, int pt_width, const int* seq_start,
                                       const int* seq_pos0, void* out, long long out_stride, int n_seqs, int q_blocks,
                                       int n_heads, int n_kv_heads, int head_dim, float scale, int window, int n_pages,
                                       int* error_flag, void* stream) {
    if (n_seqs == 0 || q_blocks == 0) return 0;
    HB_REQUIRE(hb_attention_prefill_tc_supported(n_heads, n_kv_heads, head_dim),
               "attention_prefill_tc: head size %d is not built (64, 128)", head_dim);
    HB_REQUIRE(q_blocks <= 65535 && error_flag != nullptr, "attention_prefill_tc: bad sizes");
    HB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0, "attention_prefill_tc: queries must have 16-byte aligned rows");
    HB_REQUIRE(out_stride % 8 == 0 && ((uintptr_t)out & 15) == 0, "attention_prefill_tc: output must have 16-byte aligned rows");
    HB_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0, "attention_prefill_tc: cache must be 16-byte aligned");
    CUtensorMap mq, mk, mv;
    const long long cache_rows = (long long)n_pages * n_kv_heads * HB_PAGE_TOKENS;
    if (tc_make_map(&mq, q, n_tokens, (long long)n_heads * head_dim, q_stride, FA_ROWS)) return 1;
    if (tc_make_map(&mk, k_cache, cache_rows, head_dim, head_dim, HB_PAGE_TOKENS)) return 1;
    if (tc_make_map(&mv, v_cache, cache_rows, head_dim, head_dim, HB_PAGE_TOKENS)) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    if (head_dim == 128)
        return launch_prefill_tc<128>(mq, mk, mv, page_table, pt_width, seq_start, seq_pos0, out, out_stride, n_seqs, q_blocks, n_heads,
                                      n_kv_heads, scale, window, n_pages, error_flag, st);
    return launch_prefill_tc<64>(mq, mk, mv, page_table, pt_width, seq_start, seq_pos0, out, out_stride, n_seqs, q_blocks, n_heads,
                                 n_kv_heads, scale, window, n_pages, error_flag, st);
}
