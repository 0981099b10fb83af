// tcgen05 / TMEM / TMA / mbarrier building blocks shared by the tensor-core matrix products
// (inline PTX for sm_100a), the work description of a product and the epilogue of one
// 16-column chunk of an accumulator.
#pragma once
#include <cuda.h>

#include "common.cuh"

#define TC_BM 128           // features per tile (MMA M)
#define TC_BK 64            // K per stage: 64 bf16 = one 128-byte swizzle row
#define TC_THREADS 192
#define TC_WAIT_LIMIT (1u << 24)

enum { TC_STORE_BF16 = 0, TC_STORE_F32 = 1, TC_ADD_F32 = 2, TC_SWIGLU_BF16 = 3 };

// ------------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait; returns false when it ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// fetches a tensor map (a kernel parameter) into the descriptor cache ahead of its first use
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// asks L2 to fetch a tile that a later tma_load will want
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128
// bytes, groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}


// ------------------------------------------------------------------------------- clusters (CTA pairs)
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// tile load into this CTA's shared memory whose bytes are counted on a barrier of the pair's
// leader CTA (`bar` is an address in the cluster's shared window)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Tile stores from shared memory (rows as in global memory, no swizzle); what lies outside the
// tensor is not written.  The issuing thread tracks them as bulk groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
// the same, adding the tile to what global memory holds (the addition is done at the memory side)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups still READ their shared memory
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// arrives (once the MMAs issued so far have finished) on the barrier at the same offset in
// every CTA of `cta_mask`
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(cta_mask) : "memory");
}
__host__ __device__ constexpr uint32_t instr_desc_bf16_mn(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

struct TcParams {
    void* out;
    long long ldc;
    int M, N, K;
    int up_row0;          // SWIGLU: row of W where the up rows start; -1: bands of 64 gate rows + their 64 up rows
    int tiles_m, tiles_n;
    int kb_total;         // K blocks per tile
    int stream_k;         // 0: whole tiles round-robin; 1: contiguous (tile, K block) ranges per CTA;
                          // 2: every tile cut into `split` equal K ranges, one per CTA;
                          // 3: the first tiles % grid tiles cut as in 1, then tiles / grid whole tiles per CTA
    int split;
    int max_slots;        // partial tiles per output tile in scratch (stream-K)
    float* partials;
    int* counters;
    int* error_flag;
    int cluster;          // stream_k == 2 only: the `split` CTAs of a tile are one cluster and sum through shared memory
    int packed;           // W is stored as tiles [row / 128][K block][128 rows][64 columns] (see tc_w_coords)
    int group_m;          // pair kernel: token tiles per group (see t2_tile_coords)
    // A norm between two products, folded into them (few tokens; single-CTA kernel only).
    // y = W (x * g * s) with the per-token s = rsqrt(mean(x^2) + eps) is computed as
    // s * (W bf16(x * g)): the product that WRITES x (TC_ADD_F32) also writes bf16(x * g) and,
    // per token, partial sums of x^2 (one per 32 features: slot = feature / 32); the product that
    // READS it multiplies its rows by s.  Sums and s in float32.
    const float* prep_w;  // producer: the norm's weight [N], nullptr: none; the factor is prep_offset + prep_w[f]
    float prep_offset;
    bf16* prep_out;       // [M, prep_ld]
    long long prep_ld;
    float* prep_sumsq;    // [M, sumsq_ld]
    int sumsq_ld;         // floats per token in prep_sumsq and in scale_sumsq
    const float* scale_sumsq;   // consumer: nullptr: none
    int scale_parts;      // slots per token to add
    float scale_inv_size, scale_eps;
};

// The most tokens of a product that serves a folded norm: token tiles of 16 and 32.  Measured per decode
// step, folded against norm kernels: 8B sizes batch 1 -5.7 %, batch 8 -3.6 %, batch 24 -1.3 %, batch 32
// -0.9 %, batch 48 and 64 +0.4 %; 3B sizes batch 16 -5.5 %, batch 32 -0.1 %, batch 64 +3.2 %; 1B sizes
// batch 32 -1.0 %, batch 48 -1.4 %, batch 64 0: with 64 tokens the longer epilogues of the residual
// products cost what the two kernels saved, or more.
#define TC_SCALE_ROWS 32

// The consumer's per-token factors for the tokens of a tile column block that starts at token 0
// (folding is used with one token tile only).  128 / TC_SCALE_ROWS threads per token: each adds
// its share of the groups of four partial sums, the threads of a token add up through shuffles
// in a fixed order; all loads of a thread are in flight at once, so the factors
// cost one or two round trips to L2, not one per four slots.  `srow` is shared memory of
// TC_SCALE_ROWS floats.  All 128 epilogue threads call it once.
__device__ __forceinline__ void tc_row_scales(const TcParams& p, float* srow, int et) {
    if (p.scale_sumsq == nullptr) return;
    constexpr int TPT = 128 / TC_SCALE_ROWS;           // threads per token
    const int token = et / TPT, sub = et % TPT;
    float acc = 0.0f;
    if (token < p.M) {
        const float4* src = reinterpret_cast<const float4*>(p.scale_sumsq + (size_t)token * p.sumsq_ld);
        const int groups = p.scale_parts >> 2;
        float4 t[4];
#pragma unroll 1
        for (int i0 = sub; i0 < groups; i0 += 4 * TPT) {
#pragma unroll
            for (int u = 0; u < 4; u++)
                t[u] = i0 + TPT * u < groups ? __ldcg(src + i0 + TPT * u) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 4; u++) acc += (t[u].x + t[u].y) + (t[u].z + t[u].w);
        }
        if (sub == 0)
            for (int i = p.scale_parts & ~3; i < p.scale_parts; i++) acc += __ldcg(p.scale_sumsq + (size_t)token * p.sumsq_ld + i);
    }
#pragma unroll
    for (int d = 1; d < TPT; d <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (token < p.M && sub == 0) srow[token] = rsqrtf(acc * p.scale_inv_size + p.scale_eps);
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// TMA coordinates of the box of weight rows that starts at `row`, K block kb.  Row-major W:
// column kb * 64 of row `row`.  Packed W: every 128-row x 64-column tile is one contiguous
// 16 KB piece and the K blocks of a 128-row band follow one another, so a CTA that walks
// along K reads one sequential range; seen as a matrix of 64-column rows the tile starts at
// row ((row / 128) * K blocks + kb) * 128.  A box must not straddle two bands.
__device__ __forceinline__ void tc_w_coords(const TcParams& p, int row, int kb, int& x, int& y) {
    if (p.packed) {
        x = 0;
        y = ((row >> 7) * p.kb_total + kb) * TC_BM + (row & (TC_BM - 1));
    } else {
        x = kb * TC_BK;
        y = row;
    }
}

#define TC_XCHG_BYTES (2 * 16 * 64 * 4 + 2 * 16 * 64 * 2)

// Epilogue of 16 token columns [m0 + c, m0 + c + 16) of a tile: v[j] is the accumulator of
// weight row `row` (0..127, = TMEM lane) and token column c + j.  n0 is the first output
// feature of the tile.  Called by all 128 epilogue threads (et = 0..127, q = row / 32).
template <int MODE, bool FOLD = false>
__device__ __forceinline__ void tc_emit_chunk(const TcParams& p, int m0, int n0, int c, const float (&v_in)[16], uint8_t* xchg,
                                              int q, int row, int et, const float* srow = nullptr) {
    // FOLD: the kernel variant that serves a folded norm (a variant of its own, so that the
    // others keep their registers and schedule).  The consumer side: every token's row times its factor
    float v[16];
    const bool scaled = FOLD && MODE != TC_ADD_F32 && p.scale_sumsq != nullptr;
#pragma unroll
    for (int j = 0; j < 16; j++) v[j] = (FOLD && scaled) ? v_in[j] * srow[min(m0 + c + j, p.M - 1)] : v_in[j];
    if (MODE == TC_SWIGLU_BF16) {
        // rows 0..63 of the tile are gate rows, rows 64..127 the up rows of the same
        // features: pair them through shared memory, then store 16 bytes per thread
        float* xf = (float*)xchg + ((c >> 4) & 1) * (16 * 64);
        bf16* yb = (bf16*)(xchg + 2 * 16 * 64 * 4) + ((c >> 4) & 1) * (16 * 64);
        if (q >= 2) {
#pragma unroll
            for (int j = 0; j < 16; j++) xf[j * 64 + row - 64] = v[j];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (q < 2) {
#pragma unroll
            for (int j = 0; j < 16; j++) yb[j * 64 + row] = __float2bfloat16_rn(silu_fast(v[j]) * xf[j * 64 + row]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int r = et >> 3, ch = et & 7;                 // token row of the chunk, 8-feature group
        const int m = m0 + c + r, n = n0 + ch * 8;
        if (m < p.M && n < p.N) {
            bf16* o = (bf16*)p.out + (size_t)m * p.ldc + n;
            if (n + 8 <= p.N) {
                *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(yb + r * 64 + ch * 8);
            } else {
                for (int e = 0; e < p.N - n; e++) o[e] = yb[r * 64 + ch * 8 + e];
            }
        }
    } else {
        const int f = n0 + row;
        if (FOLD && MODE == TC_ADD_F32 && p.prep_w != nullptr) {
            // the producer side of a folded norm: the new values, their products with the
            // norm's weight as bfloat16, and per token the sum of squares of this warp's 32 features
            float r[16];
            float* po = (float*)p.out + (size_t)(m0 + c) * p.ldc + f;
            const bool here = f < p.N;
#pragma unroll
            for (int j = 0; j < 16; j++) r[j] = (here && m0 + c + j < p.M) ? __ldcg(po + (size_t)j * p.ldc) : 0.0f;
            const float g = here ? p.prep_offset + __ldg(p.prep_w + f) : 0.0f;
            const int lane = et & 31;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int m = m0 + c + j;
                if (m >= p.M) break;                          // the same for the whole warp
                const float nv = here ? r[j] + v[j] : 0.0f;
                if (here) {
                    po[(size_t)j * p.ldc] = nv;
                    p.prep_out[(size_t)m * p.prep_ld + f] = __float2bfloat16_rn(nv * g);
                }
                float ss = nv * nv;
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                ss += __shfl_xor_sync(0xffffffffu, ss, 8);
                ss += __shfl_xor_sync(0xffffffffu, ss, 16);
                if (lane == 0) p.prep_sumsq[(size_t)m * p.sumsq_ld + (n0 >> 5) + q] = ss;
            }
        } else if (f < p.N) {
            if (MODE == TC_ADD_F32) {
                // all loads of the residual first, then the stores: written one by one
                // the compiler must keep each load behind the store before it
                float r[16];
                float* po = (float*)p.out + (size_t)(m0 + c) * p.ldc + f;
#pragma unroll
                for (int j = 0; j < 16; j++) r[j] = (m0 + c + j < p.M) ? __ldcg(po + (size_t)j * p.ldc) : 0.0f;
#pragma unroll
                for (int j = 0; j < 16; j++)
                    if (m0 + c + j < p.M) po[(size_t)j * p.ldc] = r[j] + v[j];
            } else {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int m = m0 + c + j;
                    if (m < p.M) {
                        const size_t o = (size_t)m * p.ldc + f;
                        if (MODE == TC_STORE_BF16) ((bf16*)p.out)[o] = __float2bfloat16_rn(v[j]);
                        else ((float*)p.out)[o] = v[j];
                    }
                }
            }
        }
    }
}

// Epilogue of a summed partial tile held in the scratch layout [token][row]: thread et
// (0..127) holds, for i = 0..BN/4-1, the four rows (et & 31) * 4 .. + 3 of token
// i * 4 + (et >> 5).  The same results as tc_emit_chunk, with 16-byte accesses.
// `res`: for TC_ADD_F32, the values of the output read ahead of time (have_res; they are then
// not read again).
template <int MODE, int BN, bool FOLD = false>
__device__ __forceinline__ void tc_emit_flat(const TcParams& p, int m0, int n0, const float4 (&acc)[BN / 4], int et,
                                             const float4 (&res)[BN / 4], bool have_res, const float* srow = nullptr) {
    const int lane = et & 31, tw = et >> 5;
    const bool scaled = FOLD && MODE != TC_ADD_F32 && p.scale_sumsq != nullptr;     // the consumer side of a folded norm
    if (FOLD && MODE == TC_ADD_F32 && p.prep_w != nullptr) {
        // The producer side of a folded norm (the host passes it only with a 16-byte aligned
        // output and N a multiple of 4): new values, their products with the norm's weight as
        // bfloat16, and the sums of squares of each 32 features (8 lanes) of a token.
        const int n = n0 + lane * 4;
        const bool here = n < p.N;
        float4 g = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (here) {
            g = __ldg(reinterpret_cast<const float4*>(p.prep_w + n));
            g = make_float4(g.x + p.prep_offset, g.y + p.prep_offset, g.z + p.prep_offset, g.w + p.prep_offset);
        }
        float4 old[BN / 4];
#pragma unroll
        for (int i = 0; i < BN / 4; i++) {
            const int m = m0 + i * 4 + tw;
            old[i] = have_res ? res[i]
                              : (here && m < p.M) ? __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)m * p.ldc + n))
                                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int i = 0; i < BN / 4; i++) {
            const int m = m0 + i * 4 + tw;                      // uniform in a warp
            if (m >= p.M) continue;
            float4 nv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (here) {
                nv = make_float4(old[i].x + acc[i].x, old[i].y + acc[i].y, old[i].z + acc[i].z, old[i].w + acc[i].w);
                *reinterpret_cast<float4*>((float*)p.out + (size_t)m * p.ldc + n) = nv;
                bf16 h[4] = {__float2bfloat16_rn(nv.x * g.x), __float2bfloat16_rn(nv.y * g.y), __float2bfloat16_rn(nv.z * g.z),
                             __float2bfloat16_rn(nv.w * g.w)};
                *reinterpret_cast<uint2*>(p.prep_out + (size_t)m * p.prep_ld + n) = *reinterpret_cast<const uint2*>(h);
            }
            float ss = (nv.x * nv.x + nv.y * nv.y) + (nv.z * nv.z + nv.w * nv.w);
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            ss += __shfl_xor_sync(0xffffffffu, ss, 4);
            if ((lane & 7) == 0) p.prep_sumsq[(size_t)m * p.sumsq_ld + (n0 >> 5) + (lane >> 3)] = ss;
        }
        return;
    }
    // TC_ADD_F32 without values read ahead: all loads of the old output first, then the stores
    // (written one by one the compiler must keep each load behind the store before it: one
    // round trip per token instead of one in all)
    float4 old[MODE == TC_ADD_F32 ? BN / 4 : 1];
    const bool old_here = MODE == TC_ADD_F32 && !have_res && (p.ldc & 3) == 0 && (((uintptr_t)p.out) & 15) == 0;
    if (MODE == TC_ADD_F32 && old_here) {
        const int n = n0 + lane * 4;
#pragma unroll
        for (int i = 0; i < BN / 4; i++) {
            const int m = m0 + i * 4 + tw;
            old[MODE == TC_ADD_F32 ? i : 0] = (m < p.M && n + 4 <= p.N)
                ? __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)m * p.ldc + n))
                : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
#pragma unroll
    for (int i = 0; i < BN / 4; i++) {
        const int m = m0 + i * 4 + tw;                      // uniform in a warp
        if (m >= p.M) continue;
        const float sc = scaled ? srow[m] : 1.0f;
        const float v[4] = {FOLD ? acc[i].x * sc : acc[i].x, FOLD ? acc[i].y * sc : acc[i].y, FOLD ? acc[i].z * sc : acc[i].z,
                            FOLD ? acc[i].w * sc : acc[i].w};
        if (MODE == TC_SWIGLU_BF16) {
            // lanes 0..15 hold gate rows 4 * lane .. + 3, lanes 16..31 the up rows of the same features
            float u[4];
#pragma unroll
            for (int e = 0; e < 4; e++) u[e] = __shfl_down_sync(0xffffffffu, v[e], 16);
            const int n = n0 + lane * 4;
            if (lane < 16 && n < p.N) {
                bf16 y[4];
#pragma unroll
                for (int e = 0; e < 4; e++) y[e] = __float2bfloat16_rn(silu_fast(v[e]) * u[e]);
                bf16* o = (bf16*)p.out + (size_t)m * p.ldc + n;
                if (n + 4 <= p.N) {
                    *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(y);
                } else {
                    for (int e = 0; e < p.N - n; e++) o[e] = y[e];
                }
            }
        } else {
            const int n = n0 + lane * 4;
            if (n >= p.N) continue;
            const size_t off = (size_t)m * p.ldc + n;
            if (MODE == TC_STORE_BF16) {
                bf16* o = (bf16*)p.out + off;
                bf16 y[4];
#pragma unroll
                for (int e = 0; e < 4; e++) y[e] = __float2bfloat16_rn(v[e]);
                if (n + 4 <= p.N && (((uintptr_t)o) & 7) == 0) {
                    *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(y);
                } else {
                    for (int e = 0; e < 4 && n + e < p.N; e++) o[e] = y[e];
                }
            } else {
                float* o = (float*)p.out + off;
                if (n + 4 <= p.N && (((uintptr_t)o) & 15) == 0) {
                    float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (MODE == TC_ADD_F32)
                        r = have_res ? res[i] : old_here ? old[MODE == TC_ADD_F32 ? i : 0] : __ldcg(reinterpret_cast<const float4*>(o));
                    *reinterpret_cast<float4*>(o) = make_float4(r.x + v[0], r.y + v[1], r.z + v[2], r.w + v[3]);
                } else {
                    for (int e = 0; e < 4 && n + e < p.N; e++) o[e] = (MODE == TC_ADD_F32 ? o[e] : 0.0f) + v[e];
                }
            }
        }
    }
}

// Tensor map of a row-major bf16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zeros outside.
int tc_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows);
// Tensor map of a row-major output [rows, cols] of float32 (elem_bytes 4) or bfloat16 (2) with
// row stride ld (elements), for stores of boxes of box_rows x box_cols elements, no swizzle.
// The base must be 16-byte aligned and ld * elem_bytes a multiple of 16.
int tc_make_out_map(CUtensorMap* map, const void* base, int elem_bytes, long long rows, long long cols, long long ld,
                    int box_rows, int box_cols);
int tc_make_weight_map(CUtensorMap* map, const void* w, long long rows, long long K, long long ld, int box_rows, int packed);
