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
// Per CTA, 192 threads, as in the single-CTA kernel:
//   warp 0     TMA producer (both CTAs): own weight rows and own token half into own shared
//              memory; the bytes of both CTAs are counted on the LEADER's full[s]
//   warp 1     tensor memory owner (both CTAs allocate together); in the leader one thread
//              issues the MMAs and commits to empty[s] / acc_full[buffer] of BOTH CTAs
//   warps 2-5  epilogue (both CTAs) on their own accumulator rows; they hand a buffer back by
//              arriving on the LEADER's acc_empty[buffer] (256 arrivals)
// Work: whole 256 x 256 tiles round-robin over the pairs (persistent), token tiles fastest so
// that neighbouring pairs share a weight tile in L2.  Epilogues as in the single-CTA kernel
// (store, residual add, SwiGLU with 64 gate + 64 up rows per CTA).
//
// Every wait is bounded; a wait that runs out sets *error_flag and both CTAs drain and leave.
#include "api.h"
#include "tcgen05.cuh"

#define T2_TOKENS 256          // tokens per pair tile (MMA N)
#define T2_HALF 128            // tokens loaded by each CTA
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
#define T2_STAGES(MODE) 6
// SwiGLU epilogue: gates and ups handed over [2][32][64] float32, products [64][64] bfloat16
#define T2_XCHG_BYTES (2 * 32 * 64 * 4 + 64 * 64 * 2)

template <int MODE, int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, const TcParams p) {
    constexpr bool SWIGLU = MODE == TC_SWIGLU_BF16;
    constexpr int FEAT = SWIGLU ? 64 : TC_BM;                     // output features per CTA
    constexpr int W_BYTES = TC_BM * TC_BK * 2;
    constexpr int XCHG = SWIGLU ? T2_XCHG_BYTES : 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* xchg = smem + STAGES * T2_STAGE_BYTES;
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
            mbar_init(acce0 + 8 * b, 256);
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
            auto load_w = [&](int s, int t, int kb) {
                const int n0 = (t / p.tiles_m) * (2 * FEAT) + (int)rank * FEAT;
                const uint32_t stage = smem_base + s * T2_STAGE_BYTES;
                int x, y;
                tc_w_coords(p, n0, kb, x, y);
                tma_load_2d_pair(stage, &map_w, lead_full0 + 8 * s, x, y);
                if (SWIGLU) {
                    tc_w_coords(p, p.up_row0 + n0, kb, x, y);
                    tma_load_2d_pair(stage + W_BYTES / 2, &map_w, lead_full0 + 8 * s, x, y);
                }
            };
            auto load_a = [&](int s, int t, int kb) {
                tma_load_2d_pair(smem_base + s * T2_STAGE_BYTES + W_BYTES, &map_a, lead_full0 + 8 * s, kb * TC_BK,
                                 (t % p.tiles_m) * T2_TOKENS + (int)rank * T2_HALF);
            };
            // weights first: no kernel of a step writes them, so they are requested before
            // waiting for the kernel in front
            int early = 0;
            if (pair < tiles) {
                early = min(p.kb_total, STAGES);
                for (int j = 0; j < early; j++) {
                    if (rank == 0) mbar_expect_tx(full0 + 8 * j, 2 * T2_STAGE_BYTES);
                    load_w(j, pair, j);
                }
            }
            pdl_wait();
            for (int j = 0; j < early; j++) load_a(j, pair, j);
            int g = 0;
            bool alive = true;
            for (int t = pair; t < tiles && alive; t += n_pairs) {
                for (int kb = 0; kb < p.kb_total; kb++, g++) {
                    if (g < early) continue;
                    const int s = g % STAGES;
                    if (!mbar_wait(empty0 + 8 * s, ((g / STAGES) & 1) ^ 1)) {
                        atomicExch(p.error_flag, 11);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * T2_STAGE_BYTES);
                    load_w(s, t, kb);
                    load_a(s, t, kb);
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
            constexpr uint32_t STAGE_STEP = T2_STAGE_BYTES >> 4, A_OFF = W_BYTES >> 4;
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
                const uint32_t acc_addr = tmem_base + buf * T2_TOKENS;
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
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int et = (warp - 2) * 32 + lane;
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
            const uint32_t lane_addr = tmem_base + buf * T2_TOKENS + ((uint32_t)(q * 32) << 16);
            const int m0 = (t % p.tiles_m) * T2_TOKENS;
            const int n0 = (t / p.tiles_m) * (2 * FEAT) + (int)rank * FEAT;
            if (MODE == TC_ADD_F32) {
                // residual add: 64 tokens at a time, all 64 old values requested before the first
                // store (16 at a time the loads' round trips, 16 per tile, outlast a short K loop)
                const int f = n0 + row;
#pragma unroll 1
                for (int c = 0; c < T2_TOKENS; c += 64) {
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
            } else if (MODE == TC_SWIGLU_BF16) {
                // 64 tokens at a time.  Rows 0..63 of this CTA's half tile are gate rows, rows
                // 64..127 the up rows of the same 64 features.  The gate threads hand the gates
                // of tokens 32..63 to the up threads and take the ups of tokens 0..31 from them
                // (through shared memory), so that all four warps share the activation; the
                // products go to shared memory as bfloat16 [token][feature] and leave with
                // 16-byte stores.  Two block barriers per 64 tokens.
                float* xf = (float*)xchg;                                  // [2][32 tokens][64 features] float32
                bf16* yb = (bf16*)(xchg + 2 * 32 * 64 * 4);                // [64 tokens][64 features]
                const bool gate_thread = row < 64;
                const int f = row & 63;
#pragma unroll 1
                for (int c = 0; c < T2_TOKENS; c += 64) {
                    if (m0 + c >= p.M) break;
                    float v[4][16];
#pragma unroll
                    for (int u = 0; u < 4; u++) tmem_ld16(lane_addr + c + 16 * u, v[u]);
                    // gates of tokens 32..63 -> xf[0], ups of tokens 0..31 -> xf[1]
                    float* mine = xf + (gate_thread ? 0 : 32 * 64);
#pragma unroll
                    for (int u = 0; u < 2; u++)
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            mine[(16 * u + j) * 64 + f] = gate_thread ? v[2 + u][j] : v[u][j];
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const float* theirs = xf + (gate_thread ? 32 * 64 : 0);
#pragma unroll
                    for (int u = 0; u < 2; u++)
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const float other = theirs[(16 * u + j) * 64 + f];
                            const float y = gate_thread ? silu_f32(v[u][j]) * other : silu_f32(other) * v[2 + u][j];
                            yb[((gate_thread ? 0 : 32) + 16 * u + j) * 64 + f] = __float2bfloat16_rn(y);
                        }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const int idx = et + 128 * k, r = idx >> 3, ch = idx & 7;     // token of the group, 8-feature piece
                        const int m = m0 + c + r, n = n0 + ch * 8;
                        if (m < p.M && n < p.N) {
                            bf16* o = (bf16*)p.out + (size_t)m * p.ldc + n;
                            if (n + 8 <= p.N) {
                                *reinterpret_cast<uint4*>(o) = *reinterpret_cast<const uint4*>(yb + r * 64 + ch * 8);
                            } else {
                                for (int e = 0; e < p.N - n; e++) o[e] = yb[r * 64 + ch * 8 + e];
                            }
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < T2_TOKENS; c += 16) {
                    if (m0 + c >= p.M) break;
                    float v[16];
                    tmem_ld16(lane_addr + c, v);
                    tc_emit_chunk<MODE>(p, m0, n0, c, v, xchg, q, row, et);
                }
            }
            tc_fence_before();
            mbar_arrive_cluster(lead_acce0 + 8 * buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // nobody leaves while the peer may still signal it or read its shared memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <int MODE>
static int launch_tc2(const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int pairs, cudaStream_t s) {
    constexpr int STAGES = T2_STAGES(MODE);
    constexpr int SMEM = STAGES * T2_STAGE_BYTES + (MODE == TC_SWIGLU_BF16 ? T2_XCHG_BYTES : 0) + (2 * STAGES + 4) * 8 + 16 + 1024;
    static_assert(SMEM <= 227 * 1024, "tile pipeline does not fit shared memory");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<MODE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("gemm_tc2: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    cudaError_t e = hb_launch(gemm_tc2_kernel<MODE, STAGES>, dim3(2 * pairs), dim3(TC_THREADS), SMEM, s, mw, ma, prm);
    if (e != cudaSuccess) return hb_fail("gemm_tc2: launch failed: %s", cudaGetErrorString(e));
    return hb_check_launch("gemm_tc2");
}

// How many CTA pairs of the kernel can be resident at once (a GPC with an odd number of SMs
// leaves one without a partner): the persistent grid must not be larger.
template <int MODE>
static int query_pairs() {
    constexpr int STAGES = T2_STAGES(MODE);
    constexpr int SMEM = STAGES * T2_STAGE_BYTES + (MODE == TC_SWIGLU_BF16 ? T2_XCHG_BYTES : 0) + (2 * STAGES + 4) * 8 + 16 + 1024;
    cudaFuncSetAttribute(gemm_tc2_kernel<MODE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    cudaLaunchConfig_t cfg = {};
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = SMEM;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_tc2_kernel<MODE, STAGES>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return clusters < sms / 2 ? clusters : sms / 2;
}
static int resident_pairs(int mode) {
    static int cached[4] = {-1, -1, -1, -1};
    if (cached[mode] < 0) {
        switch (mode) {
            case TC_STORE_BF16: cached[mode] = query_pairs<TC_STORE_BF16>(); break;
            case TC_STORE_F32: cached[mode] = query_pairs<TC_STORE_F32>(); break;
            case TC_ADD_F32: cached[mode] = query_pairs<TC_ADD_F32>(); break;
            default: cached[mode] = query_pairs<TC_SWIGLU_BF16>(); break;
        }
    }
    return cached[mode];
}
extern "C" int hb_gemm_tc2_resident_pairs(int mode) { return resident_pairs(mode & 3); }

// Whether the pair kernel should take a product: enough tokens to fill 256-token tiles.
// From 768 tokens on.  Below, a product has too few 256 x 256 tiles for 74 pairs (512 tokens x 4096
// features: 32) and the single-CTA kernel, which cuts K when tiles are few, is faster: a prompt of
// 512 tokens through 4 layers of the 8B sizes 1.64 against 1.77 ms, 768 tokens 1.92 either way,
// 1024 tokens 2.42 against 2.23 ms.
extern "C" int hb_gemm_tc2_wanted(int M, int N, int K) { return M >= 768 && N >= 256 && K >= 64; }

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
    HB_REQUIRE(!packed || mode != TC_SWIGLU_BF16 || up_row0 % 64 == 0, "gemm_tc2: packed up rows must start at a multiple of 64");
    HB_REQUIRE(error_flag != nullptr, "gemm_tc2: no error flag");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 + N <= w_rows, "gemm_tc2: up rows lie outside the weight matrix");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || (ldc % 8 == 0 && ((uintptr_t)out & 15) == 0),
               "gemm_tc2: the SwiGLU output needs 16-byte aligned rows");
    const int feat = mode == TC_SWIGLU_BF16 ? 64 : TC_BM;
    TcParams prm;
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
    const long long tiles = (long long)prm.tiles_m * prm.tiles_n;
    int pairs = resident_pairs(mode);
    if (pairs < 1) return hb_fail("gemm_tc2: no CTA pair can be resident on this device");
    if (tiles < pairs) pairs = (int)tiles;
    CUtensorMap mw, ma;
    if (tc_make_weight_map(&mw, w, w_rows, K, ldw, mode == TC_SWIGLU_BF16 ? 64 : TC_BM, packed)) return 1;
    if (tc_make_map(&ma, a, M, K, lda, T2_HALF)) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    switch (mode) {
        case TC_STORE_BF16: return launch_tc2<TC_STORE_BF16>(mw, ma, prm, pairs, s);
        case TC_STORE_F32: return launch_tc2<TC_STORE_F32>(mw, ma, prm, pairs, s);
        case TC_ADD_F32: return launch_tc2<TC_ADD_F32>(mw, ma, prm, pairs, s);
        default: return launch_tc2<TC_SWIGLU_BF16>(mw, ma, prm, pairs, s);
    }
}
