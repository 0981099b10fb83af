// Tensor-core matrix product on CTA pairs (tcgen05 cta_group::2) for many-token products:
// C[M,N] (+)= A[M,K] * W[N,K]^T, bfloat16 in, float32 accumulation in tensor memory.
//
// Two CTAs on neighbouring SMs (a cluster of 2) share one 256 x 256 output tile: CTA r holds
// 128 of the tile's 256 weight rows and 128 of its 256 tokens in shared memory; one
// tcgen05.mma.cta_group::2 (issued by the pair's leader, CTA 0) multiplies all 256 weight rows
// with all 256 tokens, each CTA accumulating its own 128 weight rows in its own tensor
// memory.  Per K block a CTA loads 32 KB for 4.2 MFLOP of its own, against 48 KB for the same
// work in the single-CTA kernel: the single-CTA kernel is bound by the bytes it pulls from L2
// at this tile size, this one is not.  No multicast loads: each CTA loads its own halves.
//
// Per CTA, 320 threads:
//   warp 0     TMA producer (both CTAs): own weight rows and own token half into own shared
//              memory; the bytes of both CTAs are counted on the LEADER's full[s].  What this
//              one thread does per K block is on the pipeline's critical path: the tile's
//              coordinates are computed once per tile, not per K block (with two integer
//              divisions per K block the whole kernel was 15 % slower)
//   warp 1     tensor memory owner (both CTAs allocate together); in the leader one thread
//              issues the MMAs and commits to empty[s] / acc_full[buffer] of BOTH CTAs
//   warps 2-9  epilogue (both CTAs), two teams of four warps (a warp reads one quarter of the
//              tensor memory's lanes) that take turns on pieces of 16 or 32 tokens of their own
//              accumulator rows: registers -> shared memory laid out as the output's rows ->
//              ONE tile store (cp.async.bulk.tensor, or cp.reduce...add for the residual add,
//              where the memory side adds) per piece.  Stores of full lines, nothing waits for
//              a load: a 128 x 256 half tile leaves in 5 to 9 us, against 11 to 24 us with one
//              element per thread and store (bfloat16 stores of 64 bytes per warp, residual
//              loads whose round trips serialise).  They hand a buffer back by arriving on the
//              LEADER's acc_empty[buffer] (512 arrivals)
// Work: whole 256 x 256 tiles round-robin over the pairs (persistent), in the order of
// t2_tile_coords.  Epilogues: store, residual add, SwiGLU with 64 gate + 64 up rows per CTA.
//
// Measured and left out: tiles of 512 tokens (two MMAs of 256 tokens per K step, 48 KB per
// stage, 0.75 of the bytes per flop): the one accumulator pair fills the tensor memory, so the
// epilogue is not hidden, and its K loop needs 0.82 us per block against 2 x 0.375 us: slower
// at every size of the 8B shape from 1024 to 8192 tokens.
//
// Every wait is bounded; a wait that runs out sets *error_flag and both CTAs drain and leave.
#include "api.h"
#include "tcgen05.cuh"

#define T2_TOKENS 256          // tokens per pair tile (MMA N)
#define T2_HALF 128            // tokens loaded by each CTA
#define T2_GROUP_TILES 8       // token tiles (2048 tokens) that are walked together (t2_tile_coords)
#define T2_STAGE_BYTES (TC_BM * TC_BK * 2 + T2_HALF * TC_BK * 2)     // 32 KB per CTA and stage
// 6 stages of 32 KB; a 7th (measured) changes nothing, and asking L2 ahead for the weight tiles
// of later K blocks (cp.async.bulk.prefetch) made the kernel slower.  Cutting the tiles of the
// last, partly filled wave over all pairs (float32 partial tiles of 128 KB per CTA in scratch,
// summed by the last contributor) was measured too: the sums cost more than the idle pairs
// (o projection at 2048 tokens: 99 us against 73 us), so tiles stay whole.
// What bounds the K loop is an SM's TMA intake: 32 KB per K block (16 KB of weights, 16 KB of
// tokens) at about 60 GB/s is 0.47 us, the four MMAs need 0.27 us.  One SM takes over 100
// GB/s from L2 through cp.async (measured with 128 KB in flight), so the token tiles were moved
// to four loader warps (cp.async into the swizzled layout, cp.async.mbarrier.arrive on a local
// barrier, a forwarder thread for the arrival on the leader's barrier): correct, but 174 us
// for the qkv product against 82 us: with six stages the chain stage free -> copies -> barrier
// -> forwarder -> MMA is twice as long as TMA's.  (A loader thread that arrives remotely
// itself waits, with the release, for all its copies in flight: 261 us.)
#define T2_STAGES 6
// Warp 0 loads, warp 1 issues the MMAs, warps 2-9 are two epilogue teams of four warps (one warp
// per quarter of the tensor memory's lanes in each).
#define T2_THREADS 320
// Shared memory of the epilogue: 16 KB per team.  Tile stores: two buffers of 8 KB ([16 tokens]
// [128 features] float32, or [32][128] bfloat16); SwiGLU: gates and ups handed over [2][16][64]
// float32, then two buffers [32 tokens][64 features] bfloat16.  The path of plain stores uses
// the first team's and the start of the second's ([2][32][64] float32 + [64][64] bfloat16).
#define T2_TEAM_BYTES (16 * 1024)
#define T2_XCHG_BYTES (2 * T2_TEAM_BYTES)

// Tile t of the persistent loop -> token tile tm, feature tile tn.  The token tiles come in
// groups of p.group_m; inside a group the token tiles run fastest (neighbouring pairs share a
// weight tile in L2), then the feature tiles, then the next group: the activations of a group
// (2048 tokens) stay in L2 while the weights stream past them, instead of all activations being
// read again for every few weight tiles (8192 tokens x 4096: 67 MB per wave of tiles).
__device__ __forceinline__ void t2_tile_coords(const TcParams& p, int t, int& tm, int& tn) {
    const int per_group = p.group_m * p.tiles_n, full = p.tiles_m / p.group_m;
    const int g = t / per_group;
    if (g < full) {
        const int local = t - g * per_group;
        tm = g * p.group_m + local % p.group_m;
        tn = local / p.group_m;
    } else {
        const int rest = p.tiles_m - full * p.group_m, local = t - full * per_group;
        tm = full * p.group_m + local % rest;
        tn = local / rest;
    }
}

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                const __grid_constant__ CUtensorMap map_o, const TcParams p, const int tma_out) {
    constexpr bool SWIGLU = MODE == TC_SWIGLU_BF16;
    constexpr int STAGES = T2_STAGES;
    constexpr int STAGE_BYTES = T2_STAGE_BYTES;
    constexpr int TOKENS = T2_TOKENS;
    constexpr int FEAT = SWIGLU ? 64 : TC_BM;                     // output features per CTA
    constexpr int W_BYTES = TC_BM * TC_BK * 2;
    constexpr int XCHG = T2_XCHG_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* xchg = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(xchg + XCHG);                    // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                      // 0: leader of the pair
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);
    // the leader's full[] and acc_empty[] as seen from this CTA
    const uint32_t lead_full0 = mapa_shared(full0, 0), lead_acce0 = mapa_shared(acce0, 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 2 * (T2_THREADS - 64));       // every epilogue thread of both CTAs
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                           // the peer's barriers exist from here on
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    const int tiles = p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            // tile coordinates once per tile: this thread's time per K block is the pipeline's
            auto load_w = [&](int s, int tn, int kb) {
                const int n0 = tn * (2 * FEAT) + (int)rank * FEAT;
                const uint32_t stage = smem_base + s * STAGE_BYTES;
                int x, y;
                tc_w_coords(p, SWIGLU && p.up_row0 < 0 ? 2 * n0 : n0, kb, x, y);       // up_row0 < 0: [gate; up] in bands, one box
                tma_load_2d_pair(stage, &map_w, lead_full0 + 8 * s, x, y);
                if (SWIGLU && p.up_row0 >= 0) {
                    tc_w_coords(p, p.up_row0 + n0, kb, x, y);
                    tma_load_2d_pair(stage + W_BYTES / 2, &map_w, lead_full0 + 8 * s, x, y);
                }
            };
            auto load_a = [&](int s, int tm, int kb) {
                tma_load_2d_pair(smem_base + s * STAGE_BYTES + W_BYTES, &map_a, lead_full0 + 8 * s, kb * TC_BK,
                                 tm * TOKENS + (int)rank * T2_HALF);
            };
            // weights first: no kernel of a step writes them, so they are requested before
            // waiting for the kernel in front
            int early = 0, tm = 0, tn = 0;
            if (pair < tiles) {
                t2_tile_coords(p, pair, tm, tn);
                early = min(p.kb_total, STAGES);
                for (int j = 0; j < early; j++) {
                    if (rank == 0) mbar_expect_tx(full0 + 8 * j, 2 * STAGE_BYTES);
                    load_w(j, tn, j);
                }
            }
            pdl_wait();
            for (int j = 0; j < early; j++) load_a(j, tm, j);
            int g = 0;
            bool alive = true;
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                t2_tile_coords(p, t, tm, tn);
                for (int kb = 0; kb < p.kb_total; kb++, g++) {
                    if (g < early) continue;
                    const int s = g % STAGES;
                    if (!mbar_wait(empty0 + 8 * s, ((g / STAGES) & 1) ^ 1)) {
                        atomicExch(p.error_flag, 11);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * STAGE_BYTES);
                    load_w(s, tn, kb);
                    load_a(s, tm, kb);
                }
            }
            // the copies into THIS CTA's shared memory must land before it may exit.  Their bytes
            // are counted on the leader's barrier, which this CTA can test only if it is the
            // leader; the cluster-wide barrier at the end covers the other CTA (the leader
            // leaves its loops only after the MMAs that consumed the data have finished).
            if (rank == 0)
                for (int i = max(0, g - STAGES); i < g; i++)
                    if (!mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1)) atomicExch(p.error_flag, 12);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_bf16_mn(256, T2_TOKENS);
            const uint64_t desc0 = smem_desc_sw128(smem_base);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            constexpr uint32_t STAGE_STEP = STAGE_BYTES >> 4, A_OFF = W_BYTES >> 4;
            int s = 0, item = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int t = pair; t < tiles && alive; t += n_pairs, item++) {
                const int buf = item & 1;
                if (!mbar_wait(acce0 + 8 * buf, ((item >> 1) & 1) ^ 1)) {
                    atomicExch(p.error_flag, 15);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t acc_addr = tmem_base + buf * TOKENS;
                for (int kb = 0; kb < p.kb_total; kb++) {
                    if (!mbar_wait(full0 + 8 * s, ph)) {
                        atomicExch(p.error_flag, 13);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t w_lo = desc_lo0 + s * STAGE_STEP;
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        const uint64_t wdesc = ((uint64_t)desc_hi << 32) | (w_lo + 2 * kk);
                        const uint64_t tdesc = ((uint64_t)desc_hi << 32) | (w_lo + A_OFF + 2 * kk);
                        umma_bf16_pair(acc_addr, wdesc, tdesc, idesc, (kb | kk) ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * s, 3);      // frees the stage in both CTAs
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                umma_commit_pair(accf0 + 8 * buf, 3);          // the item's accumulators are complete in both CTAs
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: two teams of four warps
        const int q = warp & 3;                                   // the quarter of the tensor memory's lanes this warp may read
        const int team = (warp - 2) >> 2;
        const int row = q * 32 + lane;
        const int et = ((warp - 2) & 3) * 32 + lane;              // thread of the team
        const bool issuer = et == 0;                              // issues and tracks the team's tile stores
        const int team_bar = 1 + team;
        uint8_t* stage_mem = xchg + team * T2_TEAM_BYTES;
        int issued = 0;                                           // tile stores of this team so far (chooses the buffer)
        pdl_wait();
        int item = 0;
        for (int t = pair; t < tiles; t += n_pairs, item++) {
            const int buf = item & 1;
            if (!mbar_wait(accf0 + 8 * buf, (item >> 1) & 1)) {
                atomicExch(p.error_flag, 14);
                *abort_flag = 1;
                break;
            }
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t lane_addr = tmem_base + buf * TOKENS + ((uint32_t)(q * 32) << 16);
            int tm, tn;
            t2_tile_coords(p, t, tm, tn);
            const int m0 = tm * TOKENS;
            const int n0 = tn * (2 * FEAT) + (int)rank * FEAT;
            if (tma_out) {
                // CH tokens at a time, the teams taking turns: accumulators -> registers -> shared
                // memory laid out as the output's rows -> one tile store (or tile add) by the
                // team's issuer.  Two buffers per team: a buffer is written again once the store
                // before the last has read it.
                constexpr int CH = MODE == TC_STORE_BF16 || SWIGLU ? 32 : 16;
#pragma unroll 1
                for (int c = team * CH; c < TOKENS; c += 2 * CH) {
                    if (m0 + c >= p.M) break;
                    const int b = issued & 1;
                    issued++;
                    if (issuer) bulk_wait_read<1>();
                    asm volatile("bar.sync %0, 128;" ::"r"(team_bar) : "memory");
                    if (SWIGLU) {
                        // Rows 0..63 of this CTA's half tile are gate rows, rows 64..127 the up rows
                        // of the same 64 features.  The gate threads hand the gates of tokens
                        // 16..31 to the up threads and take the ups of tokens 0..15 from them, so
                        // that all four warps share the activation.
                        float* xf = (float*)stage_mem;                               // [2][16 tokens][64 features] float32
                        bf16* yb = (bf16*)(stage_mem + 2 * 16 * 64 * 4) + b * (32 * 64);   // [32 tokens][64 features]
                        const bool gate_thread = row < 64;
                        const int f = row & 63;
                        float v[2][16];
                        tmem_ld16(lane_addr + c, v[0]);
                        tmem_ld16(lane_addr + c + 16, v[1]);
                        float* mine = xf + (gate_thread ? 0 : 16 * 64);
#pragma unroll
                        for (int j = 0; j < 16; j++) mine[j * 64 + f] = gate_thread ? v[1][j] : v[0][j];
                        asm volatile("bar.sync %0, 128;" ::"r"(team_bar) : "memory");
                        const float* theirs = xf + (gate_thread ? 16 * 64 : 0);
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const float other = theirs[j * 64 + f];
                            const float y = gate_thread ? silu_fast(v[0][j]) * other : silu_fast(other) * v[1][j];
                            yb[((gate_thread ? 0 : 16) + j) * 64 + f] = __float2bfloat16_rn(y);
                        }
                        fence_async_shared();
                        asm volatile("bar.sync %0, 128;" ::"r"(team_bar) : "memory");
                        if (issuer) {
                            tma_store_2d(&map_o, smem_u32(yb), n0, m0 + c);
                            bulk_commit();
                        }
                    } else if (MODE == TC_STORE_BF16) {
                        bf16* yb = (bf16*)stage_mem + b * (32 * TC_BM);              // [32 tokens][128 features]
                        float v[2][16];
                        tmem_ld16(lane_addr + c, v[0]);
                        tmem_ld16(lane_addr + c + 16, v[1]);
#pragma unroll
                        for (int u = 0; u < 2; u++)
#pragma unroll
                            for (int j = 0; j < 16; j++) yb[(16 * u + j) * TC_BM + row] = __float2bfloat16_rn(v[u][j]);
                        fence_async_shared();
                        asm volatile("bar.sync %0, 128;" ::"r"(team_bar) : "memory");
                        if (issuer) {
                            tma_store_2d(&map_o, smem_u32(yb), n0, m0 + c);
                            bulk_commit();
                        }
                    } else {
                        float* yf = (float*)stage_mem + b * (16 * TC_BM);            // [16 tokens][128 features]
                        float v[16];
                        tmem_ld16(lane_addr + c, v);
#pragma unroll
                        for (int j = 0; j < 16; j++) yf[j * TC_BM + row] = v[j];
                        fence_async_shared();
                        asm volatile("bar.sync %0, 128;" ::"r"(team_bar) : "memory");
                        if (issuer) {
                            if (MODE == TC_ADD_F32) tma_reduce_add_2d(&map_o, smem_u32(yf), n0, m0 + c);
                            else tma_store_2d(&map_o, smem_u32(yf), n0, m0 + c);
                            bulk_commit();
                        }
                    }
                }
            } else if (team == 0 && !SWIGLU) {
                // An output whose rows a tile store cannot address (base, row stride or row length
                // no multiple of 16 bytes): the first team writes the tile element by element.
                if (MODE == TC_ADD_F32) {
                    // residual add: 64 tokens at a time, all 64 old values requested before the first store
                    const int f = n0 + row;
#pragma unroll 1
                    for (int c = 0; c < TOKENS; c += 64) {
                        if (m0 + c >= p.M) break;
                        float v[4][16], r[4][16];
#pragma unroll
                        for (int u = 0; u < 4; u++) tmem_ld16(lane_addr + c + 16 * u, v[u]);
                        if (f < p.N) {
                            float* po = (float*)p.out + (size_t)(m0 + c) * p.ldc + f;
#pragma unroll
                            for (int u = 0; u < 4; u++)
#pragma unroll
                                for (int j = 0; j < 16; j++)
                                    r[u][j] = (m0 + c + 16 * u + j < p.M) ? __ldcg(po + (size_t)(16 * u + j) * p.ldc) : 0.0f;
#pragma unroll
                            for (int u = 0; u < 4; u++)
#pragma unroll
                                for (int j = 0; j < 16; j++)
                                    if (m0 + c + 16 * u + j < p.M) po[(size_t)(16 * u + j) * p.ldc] = r[u][j] + v[u][j];
                        }
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < TOKENS; c += 16) {
                        if (m0 + c >= p.M) break;
                        float v[16];
                        tmem_ld16(lane_addr + c, v);
                        tc_emit_chunk<MODE>(p, m0, n0, c, v, xchg, q, row, et);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(lead_acce0 + 8 * buf);
        }
        if (issuer) bulk_wait_read<0>();                          // the stores must have read this CTA's shared memory
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // nobody leaves while the peer may still signal it or read its shared memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

constexpr int T2_SMEM_BYTES = T2_STAGES * T2_STAGE_BYTES + T2_XCHG_BYTES + (2 * T2_STAGES + 4) * 8 + 16 + 1024;
static_assert(T2_SMEM_BYTES <= 227 * 1024, "tile pipeline does not fit shared memory");

template <int MODE>
static int launch_tc2(const CUtensorMap& mw, const CUtensorMap& ma, const CUtensorMap& mo, const TcParams& prm, int tma_out, int pairs,
                      cudaStream_t s) {
    constexpr int SMEM = T2_SMEM_BYTES;
    static bool attr_set[HB_MAX_DEVICES] = {};
    const int slot = hb_device_slot();
    if (!attr_set[slot]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("gemm_tc2: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set[slot] = true;
    }
    cudaError_t e = hb_launch(gemm_tc2_kernel<MODE>, dim3(2 * pairs), dim3(T2_THREADS), SMEM, s, mw, ma, mo, prm, tma_out);
    if (e != cudaSuccess) return hb_fail("gemm_tc2: launch failed: %s", cudaGetErrorString(e));
    return hb_check_launch("gemm_tc2");
}

// How many CTA pairs of the kernel can be resident at once (a GPC with an odd number of SMs
// leaves one without a partner): the persistent grid must not be larger.
template <int MODE>
static int query_pairs() {
    constexpr int SMEM = T2_SMEM_BYTES;
    cudaFuncSetAttribute(gemm_tc2_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    cudaLaunchConfig_t cfg = {};
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(T2_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc2_kernel<MODE>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters < sms / 2 ? clusters : sms / 2;
}
static int resident_pairs(int mode) {
    static int cached[HB_MAX_DEVICES][4];
    static bool known[HB_MAX_DEVICES][4] = {};
    const int slot = hb_device_slot();
    int& c = cached[slot][mode];
    if (!known[slot][mode]) {
        switch (mode) {
            case TC_STORE_BF16: c = query_pairs<TC_STORE_BF16>(); break;
            case TC_STORE_F32: c = query_pairs<TC_STORE_F32>(); break;
            case TC_ADD_F32: c = query_pairs<TC_ADD_F32>(); break;
            default: c = query_pairs<TC_SWIGLU_BF16>(); break;
        }
        known[slot][mode] = true;
    }
    return c;
}
extern "C" int hb_gemm_tc2_resident_pairs(int mode) { return resident_pairs(mode & 3); }

// Whether the pair kernel should take a product: from 256 tokens on, unless K is long and the tiles
// are few (there the single-CTA kernel, which cuts K, is faster).  Measured per product, single-CTA
// kernel / pairs, us.  8B sizes: q,k,v (K 4096) 256 tokens 34 / 32, 512 tokens 44 / 34; o (K 4096) 38 / 32,
// 40 / 34; gate/up (K 4096) 83 / 69, 122 / 103; down (K 14336; 16 pair tiles per 256 tokens) 256 tokens
// 65 / 77, 512 tokens 81 / 81, 640 tokens 107 / 83.  1B sizes at 384 tokens: q,k,v 26 / 21, o (16 tiles,
// K 2048) 32 / 23, gate/up 50 / 40, down (K 8192, 16 tiles) 42 / 50, at 1024 tokens (32 tiles) 58 / 52.
// 3B sizes, down (K 8192): 512 tokens (24 tiles) 48 / 50, 640 tokens (36 tiles) 54 / 52.  At 128 tokens
// the single-CTA kernel wins everywhere.  A prompt through 4 layers of the 8B sizes, single-CTA only
// against this rule: 256 tokens 1.22 / 1.14 ms, 384 tokens 1.51 / 1.36, 512 tokens 1.51 / 1.40 (with the
// down projection on pairs at 512 tokens, 32 tiles: 1.44; hence 40 tiles).
extern "C" int hb_gemm_tc2_wanted(int M, int N, int K) {
    if (M < 256 || N < 256 || K < 64) return 0;
    const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    return K <= 4096 || tiles >= 40;
}

// Arguments as hb_gemm_tc (no scratch: whole tiles only).
extern "C" int hb_gemm_tc2(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out,
                           long long ldc, int M, int N, int K, int mode, int up_row0, int* error_flag, int packed, void* stream) {
    if (M == 0 || N == 0) return 0;
    HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc2: bad sizes M=%d N=%d K=%d", M, N, K);
    HB_REQUIRE(mode >= 0 && mode <= 3, "gemm_tc2: unknown epilogue %d", mode);
    HB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc2: operands must be 16-byte aligned");
    HB_REQUIRE(lda % 8 == 0 && (packed || ldw % 8 == 0), "gemm_tc2: row strides %lld and %lld must be multiples of 8 elements", lda, ldw);
    HB_REQUIRE(lda >= K && (packed || ldw >= K) && ldc >= N, "gemm_tc2: a row stride is smaller than its row");
    HB_REQUIRE(!packed || N <= w_rows, "gemm_tc2: %d output features from a packed matrix of %lld rows", N, w_rows);
    HB_REQUIRE(!packed || mode != TC_SWIGLU_BF16 || up_row0 % 64 == 0 || up_row0 == -1, "gemm_tc2: packed up rows must start at a multiple of 64");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 >= -1, "gemm_tc2: up rows start at %d", up_row0);
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 != -1 || (N % 64 == 0 && 2LL * N <= w_rows),
               "gemm_tc2: [gate; up] in bands needs a multiple of 64 features and both halves in the matrix");
    HB_REQUIRE(error_flag != nullptr, "gemm_tc2: no error flag");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 < 0 || up_row0 + N <= w_rows, "gemm_tc2: up rows lie outside the weight matrix");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || (ldc % 8 == 0 && N % 8 == 0 && ((uintptr_t)out & 15) == 0),
               "gemm_tc2: the SwiGLU output needs 16-byte aligned rows of a multiple of 8 features (the single-CTA kernel takes others)");
    const int feat = mode == TC_SWIGLU_BF16 ? 64 : TC_BM;
    TcParams prm = {};
    prm.out = out;
    prm.ldc = ldc;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.up_row0 = up_row0;
    prm.tiles_m = (M + T2_TOKENS - 1) / T2_TOKENS;
    prm.tiles_n = (N + 2 * feat - 1) / (2 * feat);
    prm.kb_total = (K + TC_BK - 1) / TC_BK;
    prm.stream_k = 0;
    prm.split = 1;
    prm.max_slots = 0;
    prm.partials = nullptr;
    prm.counters = nullptr;
    prm.error_flag = error_flag;
    prm.packed = packed ? 1 : 0;
    prm.group_m = T2_GROUP_TILES;
    const long long tiles = (long long)prm.tiles_m * prm.tiles_n;
    int pairs = resident_pairs(mode);
    if (pairs < 1) return hb_fail("gemm_tc2: no CTA pair can be resident on this device");
    if (tiles < pairs) pairs = (int)tiles;
    // Tile stores need a 16-byte aligned base and row stride, and rows of a multiple of 16 bytes:
    // a store that the tensor's edge cuts is cut at a 16-byte boundary, not at the last element
    // (seen with bfloat16 rows of 1100 elements: the four elements behind each row were written).
    // Other outputs are written with plain stores.
    const int elem = (mode == TC_STORE_BF16 || mode == TC_SWIGLU_BF16) ? 2 : 4;
    const int tma_out = ((uintptr_t)out & 15) == 0 && (ldc * elem) % 16 == 0 && ((long long)N * elem) % 16 == 0;
    CUtensorMap mw, ma, mo;
    if (tma_out) {
        if (tc_make_out_map(&mo, out, elem, M, N, ldc, elem == 4 ? 16 : 32, feat)) return 1;
    } else {
        memset(&mo, 0, sizeof(mo));
    }
    if (tc_make_weight_map(&mw, w, w_rows, K, ldw, mode == TC_SWIGLU_BF16 && up_row0 >= 0 ? 64 : TC_BM, packed)) return 1;
    if (tc_make_map(&ma, a, M, K, lda, T2_HALF)) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    switch (mode) {
        case TC_STORE_BF16: return launch_tc2<TC_STORE_BF16>(mw, ma, mo, prm, tma_out, pairs, s);
        case TC_STORE_F32: return launch_tc2<TC_STORE_F32>(mw, ma, mo, prm, tma_out, pairs, s);
        case TC_ADD_F32: return launch_tc2<TC_ADD_F32>(mw, ma, mo, prm, tma_out, pairs, s);
        default: return launch_tc2<TC_SWIGLU_BF16>(mw, ma, mo, prm, tma_out, pairs, s);
    }
}
