// The tensor-core matrix product's kernel template and its launch helpers, shared by the two
// translation units that instantiate it (gemm_tc.cu: token tiles 16 and 32; gemm_tc_wide.cu: 64,
// 128 and 256), so that they compile side by side.  The scheme is described in gemm_tc.cu.
#pragma once
#include "api.h"
#include "tcgen05.cuh"

template <int BN, int MODE>
struct TcLayout {
    static constexpr bool SWIGLU = MODE == TC_SWIGLU_BF16;
    static constexpr int FEAT = SWIGLU ? 64 : TC_BM;                   // output features per tile
    static constexpr int W_BYTES = TC_BM * TC_BK * 2;                  // 16 KB: 128 weight rows
    static constexpr int A_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    static constexpr int NBUF = 2;                                     // accumulator buffers
    static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
    static constexpr int XCHG_BYTES = SWIGLU ? TC_XCHG_BYTES : 0;
    static constexpr int PART_BYTES = BN * TC_BM * 4;                  // one partial tile, float32 [token][row]
};
#define TC_MAX_CLUSTER 8        // portable cluster size: the most K ranges a tile is cut into in cluster mode

// The work items of one CTA, in order: (tile, first K block, end K block).
struct TcSchedule {
    int tiles, kbt, stream_k, split, per;
    int cur, end, step;       // stream-K: unit cursor and range end; tiles: tile cursor and stride
    long long base;
    int rem, grid, cta;
    int whole_left, whole_next;   // mode 3: whole tiles still to come and the next one
    __device__ __forceinline__ void init(const TcParams& p) {
        tiles = p.tiles_m * p.tiles_n;
        kbt = p.kb_total;
        stream_k = p.stream_k;
        split = p.split;
        grid = gridDim.x;
        cta = blockIdx.x;
        if (stream_k == 2) {
            per = (kbt + split - 1) / split;
            const int t = cta / split, part = cta - t * split;
            cur = t * kbt + part * per;                       // as a unit range of the flat space
            end = t * kbt + min(kbt, (part + 1) * per);
            if (t >= tiles) end = cur;
        } else if (stream_k) {
            // mode 3: the first tiles % grid tiles are cut like mode 1, then every CTA takes
            // tiles / grid whole tiles, so that the kernel ends with plain epilogues and the
            // sums of the cut tiles happen while the whole tiles stream
            whole_left = stream_k == 3 ? tiles / grid : 0;
            const int cut_tiles = tiles - whole_left * grid;
            whole_next = cut_tiles + cta;
            const long long units = (long long)cut_tiles * kbt;
            base = units / grid;
            rem = (int)(units % grid);
            const long long b = cta;
            cur = (int)(b * base + (b < rem ? b : rem));
            end = cur + (int)base + (b < rem ? 1 : 0);
        } else {
            cur = cta;
            step = grid;
            end = tiles;
        }
    }
    __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1) {
        if (stream_k == 3 && cur >= end) {
            if (whole_left <= 0) return false;
            tile = whole_next;
            kb0 = 0;
            kb1 = kbt;
            whole_next += grid;
            whole_left--;
            return true;
        }
        if (cur >= end) return false;
        if (stream_k) {
            tile = cur / kbt;
            kb0 = cur - tile * kbt;
            kb1 = min(kbt, kb0 + (end - cur));
            cur += kb1 - kb0;
        } else {
            tile = cur;
            kb0 = 0;
            kb1 = kbt;
            cur += step;
        }
        return true;
    }
    // stream-K: the CTA that holds work unit u
    __device__ __forceinline__ int cta_of(long long u) const {
        const long long big = (long long)rem * (base + 1);
        return u < big ? (int)(u / (base + 1)) : rem + (int)((u - big) / base);
    }
    // how many CTAs contribute to `tile` and which of them this CTA is (in K order)
    __device__ __forceinline__ void contributors(int tile, int& n, int& slot) const {
        if (stream_k == 2) {
            n = (kbt + per - 1) / per;
            slot = cta - tile * split;
        } else {
            const long long u0 = (long long)tile * kbt;
            const int c_lo = cta_of(u0);
            n = cta_of(u0 + kbt - 1) - c_lo + 1;
            slot = cta - c_lo;
        }
    }
};

// ------------------------------------------------------------------------------- kernel
// TL_EVENT(code) marks exist in timeline builds only (common.cuh): 1 predecessors finished
// (producer), 2 first stage full (MMA thread), 3 last MMA of a work item committed, 4 accumulator
// full (epilogue), 5 partial tile written and fenced, 6 tile counter known, 7 tile emitted,
// 8 block end (in a cluster's first CTA: 5 behind the last cluster barrier, 6 partial tiles summed).
//
// CLUSTER (up to 64 tokens, every tile cut into `split` <= 8 equal K ranges): the CTAs of a tile
// are one thread-block cluster.  Each writes its partial tile into the shared memory of the
// cluster's first CTA (st.shared::cluster), one cluster barrier later that CTA sums the partial
// tiles in K order and runs the epilogue: no scratch in global memory, no fence, no counter.
// With 16 tokens the partial tiles have a region of their own; with 32 and 64 they lie over
// the first CTA's pipeline stages, which a first cluster barrier declares free (every CTA's
// MMAs have finished).
// FOLD: the variant that serves a norm folded into the products around it (TcParams); launched
// only when a call asks for it, so that the plain variants keep their registers and schedule.
template <int BN, int MODE, int STAGES, bool CLUSTER, bool FOLD = false>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const TcParams p) {
    using L = TcLayout<BN, MODE>;
    constexpr bool SWIGLU = L::SWIGLU;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* xchg = smem + STAGES * L::STAGE_BYTES;
    // CLUSTER: partial tiles [part][token][row] in the first CTA's shared memory: a region of
    // their own (16 tokens), or over its pipeline stages (more tokens: no room beside them)
    constexpr bool RING = CLUSTER && BN > 16;
    uint8_t* xpart = RING ? smem : xchg + L::XCHG_BYTES;
    uint64_t* bars = (uint64_t*)(xchg + L::XCHG_BYTES + (CLUSTER && !RING ? TC_MAX_CLUSTER * L::PART_BYTES : 0));   // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* last_flag = (int*)(tmem_slot + 2);
    float* srow = (float*)(tmem_slot + 4);         // a folded norm's per-token factors (tc_row_scales), TC_SCALE_ROWS floats

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);

    TcSchedule sched;
    sched.init(p);
    int tile, kb0, kb1;
    // n0: the tile's first feature, m0: its first token (computed once per work item: the
    // producer's instructions per K block are on the pipeline's critical path)
    auto load_w = [&](int s, int n0, int kb) {
        const uint32_t stage = smem_base + s * L::STAGE_BYTES;
        int x, y;
        // [gate; up] in bands (up_row0 < 0): the 64 gate rows and the 64 up rows of the tile's
        // features are one 128-row band, one box
        tc_w_coords(p, SWIGLU && p.up_row0 < 0 ? 2 * n0 : n0, kb, x, y);
        tma_load_2d(stage, &map_w, full0 + 8 * s, x, y);
        if (SWIGLU && p.up_row0 >= 0) {
            tc_w_coords(p, p.up_row0 + n0, kb, x, y);
            tma_load_2d(stage + L::W_BYTES / 2, &map_w, full0 + 8 * s, x, y);
        }
    };
    auto load_a = [&](int s, int m0, int kb) {
        tma_load_2d(smem_base + s * L::STAGE_BYTES + L::W_BYTES, &map_a, full0 + 8 * s, kb * TC_BK, m0);
    };

    int early = 0;              // K blocks whose weight tiles thread 0 requests right away
    if (threadIdx.x == 0) {
        tma_prefetch_map(&map_w);
        tma_prefetch_map(&map_a);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < L::NBUF; b++) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 128);
        }
        *abort_flag = 0;
        *last_flag = 0;
        TL_INIT();
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // The weights are written by no kernel of a step: the first stages' weight tiles are
        // requested at once, before the block has its tensor memory and before the kernel in
        // front, whose output is only the activation operand, has finished.
        TcSchedule peek = sched;
        if (peek.next(tile, kb0, kb1)) {
            early = min(kb1 - kb0, STAGES);
            for (int j = 0; j < early; j++) {
                mbar_expect_tx(full0 + 8 * j, L::STAGE_BYTES);
                load_w(j, (tile / p.tiles_m) * L::FEAT, kb0 + j);
            }
        }
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), L::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    // CLUSTER: what the first CTA's epilogue threads carry across the cluster barrier
    constexpr int CL_NV = BN <= 64 ? BN / 4 : 1;
    float4 cl_res[CL_NV];
    float cl_row[CLUSTER && BN > 16 ? BN : 16];    // RING: this thread's weight row of the partial tile, all tokens
    int cl_m0 = 0, cl_n0 = 0;
    bool cl_have_res = false, cl_done = false;
    const int et = (warp - 2) * 32 + lane;         // 0..127 among the epilogue threads (warps 2..5)

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            pdl_wait();
            TL_EVENT(1);
            for (int j = 0; j < early; j++) load_a(j, (tile % p.tiles_m) * BN, kb0 + j);
            int g = 0;                    // K blocks issued so far (all work items)
            bool alive = true;
            while (alive && sched.next(tile, kb0, kb1)) {
                const int n0 = (tile / p.tiles_m) * L::FEAT, m0 = (tile % p.tiles_m) * BN;
                for (int kb = kb0; kb < kb1; kb++, g++) {
                    if (g < early) continue;
                    const int s = g % STAGES;
                    if (!mbar_wait(empty0 + 8 * s, ((g / STAGES) & 1) ^ 1)) {
                        atomicExch(p.error_flag, 1);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                    load_w(s, n0, kb);
                    load_a(s, m0, kb);
                }
            }
            // copies in flight must land before the CTA may exit: wait (bounded) for the
            // stages armed last; a stage the MMA thread already consumed answers at once
            for (int i = max(0, g - STAGES); i < g; i++)
                if (!mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1)) atomicExch(p.error_flag, 2);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // One thread issues every MMA, so its instruction stream is the critical path for
        // few-token tiles: descriptors advance with one 32-bit add per MMA (the high word is
        // constant) and nothing else is recomputed inside the loop.
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            const uint64_t desc0 = smem_desc_sw128(smem_base);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            constexpr uint32_t STAGE_STEP = L::STAGE_BYTES >> 4, A_OFF = L::W_BYTES >> 4;
            int s = 0, item = 0;
            uint32_t ph = 0;
            bool alive = true;
            while (alive && sched.next(tile, kb0, kb1)) {
                const int buf = item & 1;
                if (!mbar_wait(acce0 + 8 * buf, ((item >> 1) & 1) ^ 1)) {
                    atomicExch(p.error_flag, 5);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + buf * BN;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(full0 + 8 * s, ph)) {
                        atomicExch(p.error_flag, 3);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    if (item == 0 && kb == kb0) TL_EVENT(2);
                    const uint32_t w_lo = desc_lo0 + s * STAGE_STEP;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        const uint64_t wdesc = ((uint64_t)desc_hi << 32) | (w_lo + 2 * kk);
                        const uint64_t tdesc = ((uint64_t)desc_hi << 32) | (w_lo + A_OFF + 2 * kk);
                        umma_bf16(acc_addr, wdesc, tdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty0 + 8 * s);      // frees the stage when these MMAs have read it
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                umma_commit(accf0 + 8 * buf);          // arrives when the item's MMAs have finished
                TL_EVENT(3);
                item++;
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;             // weight row of the tile = TMEM lane
        pdl_wait();                                // the output, the scratch and the counters belong to earlier kernels until now
        if (FOLD) tc_row_scales(p, srow, et);      // (while the first accumulator is still being computed)
        int item = 0;
        while (sched.next(tile, kb0, kb1)) {
            const int buf = item & 1;
            if (!mbar_wait(accf0 + 8 * buf, (item >> 1) & 1)) {
                atomicExch(p.error_flag, 4);
                *abort_flag = 1;
                break;
            }
            if (*abort_flag) break;
            tc_fence_after();
            if (et == 0) TL_EVENT(4);
            const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
            const int m0 = (tile % p.tiles_m) * BN, n0 = (tile / p.tiles_m) * L::FEAT;
            const bool whole = kb0 == 0 && kb1 == p.kb_total;
            bool finish = whole;
            int contributors = 1;
            // TC_ADD_F32 with a split tile: the output's old values are requested now, by every
            // contributor, so that the one that turns out to be last need not wait for them
            // (nobody writes the tile before all contributors have counted themselves in)
            constexpr int NV = BN <= 64 ? BN / 4 : 16;
            // (Not for 64 tokens: in the cluster variant, where the first CTA's residual add takes
            // 6-9 us behind the second barrier, reading its 16 float4 ahead made a step at batch
            // 64 1.5-2 % slower, measured on one GPU in alternating runs.)
            constexpr bool RES_AHEAD = MODE == TC_ADD_F32 && BN <= 32;
            float4 res[NV];
            const bool have_res = RES_AHEAD && !whole && (p.ldc & 3) == 0 && (p.N & 3) == 0 && ((uintptr_t)p.out & 15) == 0;
            if (RES_AHEAD && have_res) {
                const int n = n0 + (et & 31) * 4;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    const int m = m0 + i * 4 + (et >> 5);
                    res[i] = (m < p.M && n < p.N) ? __ldcg(reinterpret_cast<const float4*>((const float*)p.out + (size_t)m * p.ldc + n))
                                                  : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
            if (CLUSTER) {
                cl_m0 = m0;
                cl_n0 = n0;
                cl_have_res = have_res;
#pragma unroll
                for (int i = 0; i < NV; i++) cl_res[i] = res[i];
                if (RING) {
                    // this CTA's row of the partial tile stays in registers until the first
                    // CTA's pipeline is free (the first cluster barrier, below)
#pragma unroll
                    for (int c = 0; c < BN; c += 16) tmem_ld16(lane_addr + c, *reinterpret_cast<float(*)[16]>(cl_row + (RING ? c : 0)));
                } else {
                    // partial tile into the first CTA's shared memory, slot = this CTA's K range
                    const uint32_t dst = mapa_shared(smem_u32(xpart) + (blockIdx.x % p.split) * L::PART_BYTES, 0);
#pragma unroll 1
                    for (int c = 0; c < BN; c += 16) {
                        float v[16];
                        tmem_ld16(lane_addr + c, v);
#pragma unroll
                        for (int j = 0; j < 16; j++) st_cluster_f32(dst + ((c + j) * TC_BM + row) * 4, v[j]);
                    }
                }
                tc_fence_before();
                mbar_arrive(acce0 + 8 * buf);
                cl_done = true;
                item++;
                continue;
            }
            if (!whole) {
                // partial tile to scratch: [tile][slot][token][row], float32
                int slot;
                sched.contributors(tile, contributors, slot);
                float* dst = p.partials + ((size_t)tile * p.max_slots + slot) * (size_t)(BN * TC_BM);
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    float v[16];
                    tmem_ld16(lane_addr + c, v);
#pragma unroll
                    for (int j = 0; j < 16; j++) dst[(size_t)(c + j) * TC_BM + row] = v[j];
                }
                tc_fence_before();
                mbar_arrive(acce0 + 8 * buf);                  // the accumulator buffer is free again
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) TL_EVENT(5);
                if (et == 0) {
                    const int prev = atomicAdd(p.counters + tile, 1);
                    const int last = (prev == contributors - 1) ? 1 : 0;
                    if (last) p.counters[tile] = 0;            // ready for the next launch
                    *last_flag = last;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finish = *last_flag != 0;
                __threadfence();
                if (et == 0) TL_EVENT(6);
            }
            if (finish && !whole) {
                // Sum of the partial tiles in K order with 16-byte loads: every load of one
                // contributor is in flight at once, so the sum costs one L2 round trip per
                // contributor (two are overlapped) instead of one per 16 tokens of each.
                // Token tiles above 64 go in groups of 64 tokens (registers).
                constexpr int GROUP = BN <= 64 ? BN : 64, GV = GROUP / 4;
                const int tw = et >> 5;
#pragma unroll 1
                for (int g0 = 0; g0 < BN; g0 += GROUP) {
                    if (m0 + g0 >= p.M) break;
                    const float4* src4 = reinterpret_cast<const float4*>(p.partials + (size_t)tile * p.max_slots * (size_t)(BN * TC_BM) +
                                                                         (size_t)g0 * TC_BM) + et;
                    float4 acc[GV];
#pragma unroll
                    for (int i = 0; i < GV; i++) acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
                    for (int z = 0; z < contributors; z++) {
                        const float4* pz = src4 + (size_t)z * (BN * TC_BM / 4);
                        float4 t[GV];
#pragma unroll
                        for (int i = 0; i < GV; i++)
                            t[i] = (m0 + g0 + i * 4 + tw < p.M) ? __ldcg(pz + i * TC_BM) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                        for (int i = 0; i < GV; i++) {
                            acc[i].x += t[i].x;
                            acc[i].y += t[i].y;
                            acc[i].z += t[i].z;
                            acc[i].w += t[i].w;
                        }
                    }
                    tc_emit_flat<MODE, GROUP, FOLD>(p, m0 + g0, n0, acc, et, res, have_res, srow);     // read ahead: one group only
                }
            } else if (finish) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 16) {
                    if (m0 + c >= p.M) break;
                    float v[16];
                    tmem_ld16(lane_addr + c, v);
                    tc_emit_chunk<MODE, FOLD>(p, m0, n0, c, v, xchg, q, row, et, srow);
                }
            }
            if (whole) {
                tc_fence_before();
                mbar_arrive(acce0 + 8 * buf);
            }
            if (et == 0 && finish) TL_EVENT(7);
            item++;
        }
    }
    if (CLUSTER) {
        // Every thread of every CTA of the cluster gets here exactly once (the loops above are
        // left by `break`, never by `return`).  RING: after a first barrier every CTA's copies
        // have landed and its MMAs have finished (its epilogue threads have read the
        // accumulator), so the first CTA's stages can take the partial tiles.  After the
        // (second) barrier the partial tiles of all K ranges lie in the first CTA's shared memory.
        if (RING) {
            cluster_sync_all();
            if (warp >= 2 && cl_done) {
                const int q = warp & 3, row = q * 32 + lane;
                const uint32_t dst = mapa_shared(smem_u32(xpart) + (blockIdx.x % p.split) * L::PART_BYTES, 0);
#pragma unroll
                for (int c = 0; c < (RING ? BN : 1); c++) st_cluster_f32(dst + (c * TC_BM + row) * 4, cl_row[c]);
            }
        }
        cluster_sync_all();
        if (warp >= 2 && blockIdx.x % p.split == 0 && cl_done && !*abort_flag) {
            const int parts = (p.kb_total + ((p.kb_total + p.split - 1) / p.split) - 1) / ((p.kb_total + p.split - 1) / p.split);
            if (et == 0) TL_EVENT(5);
            float4 acc[CL_NV];
#pragma unroll
            for (int i = 0; i < CL_NV; i++) acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int z = 0; z < parts; z++) {
                const float4* pz = reinterpret_cast<const float4*>(xpart + z * L::PART_BYTES) + et;
#pragma unroll
                for (int i = 0; i < CL_NV; i++) {
                    const float4 t = pz[i * TC_BM];
                    acc[i].x += t.x;
                    acc[i].y += t.y;
                    acc[i].z += t.z;
                    acc[i].w += t.w;
                }
            }
            if (et == 0) TL_EVENT(6);
            tc_emit_flat<MODE, BN <= 64 ? BN : 4, FOLD>(p, cl_m0, cl_n0, acc, et, cl_res, cl_have_res, srow);
            if (et == 0) TL_EVENT(7);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
        TL_EVENT(8);
        TL_FLUSH();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

template <int BN, int MODE, int STAGES, bool CLUSTER, bool FOLD = false>
struct TcLaunch {
    using L = TcLayout<BN, MODE>;
    static constexpr int SMEM = STAGES * L::STAGE_BYTES + L::XCHG_BYTES + (CLUSTER && BN == 16 ? TC_MAX_CLUSTER * L::PART_BYTES : 0) +
                                (2 * STAGES + 4) * 8 + 16 + (FOLD ? TC_SCALE_ROWS * 4 : 0) + 1024;
    // CLUSTER: the most K ranges of a tile: what fits over the first CTA's stages (above 16 tokens)
    static constexpr int MAX_PARTS = BN == 16 || STAGES * L::STAGE_BYTES / L::PART_BYTES >= TC_MAX_CLUSTER
                                         ? TC_MAX_CLUSTER : STAGES * L::STAGE_BYTES / L::PART_BYTES;
    static_assert(SMEM <= 227 * 1024, "tile pipeline does not fit shared memory");
    static int prepare() {
        static bool attr_set = false;
        if (!attr_set) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, STAGES, CLUSTER, FOLD>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
            if (e != cudaSuccess) return hb_fail("gemm_tc: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
            attr_set = true;
        }
        return 0;
    }
    static int launch(const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid, cudaStream_t s) {
        if (prepare()) return 1;
        cudaError_t e = CLUSTER ? hb_launch_clusters(gemm_tc_kernel<BN, MODE, STAGES, CLUSTER, FOLD>, dim3(grid), dim3(TC_THREADS), SMEM, s,
                                                     (unsigned)prm.split, mw, ma, prm)
                                : hb_launch(gemm_tc_kernel<BN, MODE, STAGES, CLUSTER, FOLD>, dim3(grid), dim3(TC_THREADS), SMEM, s, mw, ma, prm);
        if (e != cudaSuccess) return hb_fail("gemm_tc: launch failed: %s", cudaGetErrorString(e));
        return hb_check_launch("gemm_tc");
    }
    // how many clusters of `size` CTAs can be resident at once (0: the query failed)
    static int resident_clusters(int size) {
        if (prepare()) return 0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(size * 1024);
        cfg.blockDim = dim3(TC_THREADS);
        cfg.dynamicSmemBytes = SMEM;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = size;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<BN, MODE, STAGES, CLUSTER, FOLD>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            return 0;
        }
        return n;
    }
};

// The cluster variants.  16 tokens: fewer stages, room for the partial tiles beside them (a
// step of 8 layers at batch 8: 1305 us; with the partial tiles over 11 stages and the second
// cluster barrier that needs: 1327 us).  32 and 64 tokens: the stages of the plain kernels.
template <int BN, int MODE, bool FOLD = false>
using TcClusterLaunch = TcLaunch<BN, MODE, BN == 16 ? (MODE == TC_SWIGLU_BF16 ? 7 : 8) : BN == 32 ? 10 : 8, true, FOLD>;

template <int BN, int MODE>
static bool clusters_fit(int size, long long tiles) {
    static int cached[TC_MAX_CLUSTER + 1] = {0};      // 0: not asked yet, -1: none
    if (size < 2 || size > TcClusterLaunch<BN, MODE>::MAX_PARTS) return false;
    if (cached[size] == 0) {
        const int n = TcClusterLaunch<BN, MODE>::resident_clusters(size);
        cached[size] = n > 0 ? n : -1;
    }
    return cached[size] >= tiles;
}

template <int BN>
static bool clusters_fit_bn(int mode, int size, long long tiles) {
    switch (mode & 3) {
        case TC_STORE_BF16: return clusters_fit<BN, TC_STORE_BF16>(size, tiles);
        case TC_STORE_F32: return clusters_fit<BN, TC_STORE_F32>(size, tiles);
        case TC_ADD_F32: return clusters_fit<BN, TC_ADD_F32>(size, tiles);
        default: return clusters_fit<BN, TC_SWIGLU_BF16>(size, tiles);
    }
}

// One token tile, every epilogue: the cluster variant or the plain one with `STAGES` stages;
// the variants that serve a folded norm when the call brings one (up to 64 tokens).
template <int BN, int STAGES, bool FOLD>
static int tc_launch_bn_fold(bool cluster, int mode, const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid,
                             cudaStream_t s) {
    if (cluster) {
        if constexpr (BN <= 64) {
            switch (mode & 3) {
                case TC_STORE_BF16: return TcClusterLaunch<BN, TC_STORE_BF16, FOLD>::launch(mw, ma, prm, grid, s);
                case TC_STORE_F32: return TcClusterLaunch<BN, TC_STORE_F32, FOLD>::launch(mw, ma, prm, grid, s);
                case TC_ADD_F32: return TcClusterLaunch<BN, TC_ADD_F32, FOLD>::launch(mw, ma, prm, grid, s);
                default: return TcClusterLaunch<BN, TC_SWIGLU_BF16, FOLD>::launch(mw, ma, prm, grid, s);
            }
        } else {
            return hb_fail("gemm_tc: no cluster variant for token tile %d", BN);
        }
    }
    switch (mode & 3) {
        case TC_STORE_BF16: return TcLaunch<BN, TC_STORE_BF16, STAGES, false, FOLD>::launch(mw, ma, prm, grid, s);
        case TC_STORE_F32: return TcLaunch<BN, TC_STORE_F32, STAGES, false, FOLD>::launch(mw, ma, prm, grid, s);
        case TC_ADD_F32: return TcLaunch<BN, TC_ADD_F32, STAGES, false, FOLD>::launch(mw, ma, prm, grid, s);
        default: return TcLaunch<BN, TC_SWIGLU_BF16, STAGES, false, FOLD>::launch(mw, ma, prm, grid, s);
    }
}

template <int BN, int STAGES>
static int tc_launch_bn(bool cluster, int mode, const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid,
                        cudaStream_t s) {
    if (prm.prep_w != nullptr || prm.scale_sumsq != nullptr) {
        if constexpr (BN <= TC_SCALE_ROWS) return tc_launch_bn_fold<BN, STAGES, true>(cluster, mode, mw, ma, prm, grid, s);
        else return hb_fail("gemm_tc: a folded norm with a token tile of %d", BN);
    }
    return tc_launch_bn_fold<BN, STAGES, false>(cluster, mode, mw, ma, prm, grid, s);
}

// Token tiles 64, 128 and 256 live in gemm_tc_wide.cu.
int tc_wide_launch(int bn, bool cluster, int mode, const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid,
                   cudaStream_t s);
bool tc_wide_clusters_fit(int bn, int mode, int size, long long tiles);
