// A chain of few-token operations in ONE persistent launch: matrix products (the tcgen05
// product of gemm_tc.cu with each of its epilogues) and RMSNorms, run one after another by
// the same CTAs with a grid-wide barrier between two of them.
//
// Why.  A decode step of up to 64 tokens is a stream of weights: every product reads its
// matrix once, and what the device can do is bounded by how steadily that stream runs.  As
// separate launches every operation ends with a tail (partial tiles summed, the output
// written) and starts with an empty pipeline, and the next kernel's blocks cannot even be
// resident before the last one's have left (shared memory); a layer is eight such seams.
// Here one CTA per SM stays resident across the operations of a chain (output projection ->
// norm -> gate/up with SiLU -> down -> norm -> q/k/v of the next layer, six phases), and
// its TMA thread runs AHEAD of the grid barrier: weights are written by no operation, so the
// weight tiles of the next product are requested into every free stage while the current
// product's tail, the barrier and a norm between them are still under way.  Only the
// activation tile of a stage has to wait for the barrier.  The reference launches one kernel
// per operation and synchronises once per forward pass (cleanroom-transformer/src/cuda_backend.cu:
// 783-887); its one-token fusion of gate, up and SiLU (cuda_backend.cu:551-559) is the same
// idea on a smaller scale.
//
// Roles in a CTA (192 threads), as in gemm_tc.cu: warp 0 one TMA thread, warp 1 one MMA
// thread and the owner of tensor memory, warps 2-5 the epilogue (accumulator -> output; the
// partial tiles of a tile whose K range is cut, summed in K order by its last contributor:
// a fixed order) and the norms (CTA r normalises row r).  Work split of a product: with as
// many tiles as CTAs or more, tiles % CTAs tiles are cut over all CTAs first and whole tiles
// follow; with fewer, the (tile, K block) space is cut into one contiguous range per CTA.
//
// The grid barrier is a counter in global memory: one arrival per CTA and phase (release),
// a bounded spin on it (acquire).  All CTAs are resident at once because the grid is no
// larger than what the occupancy query says fits (checked on the host, which refuses
// otherwise) and nothing launched behind this kernel can take an SM before every CTA of it
// runs (dependents start only after every CTA has passed its launch_dependents).  The last
// arrival of a launch puts the counter back to zero.  Every wait is bounded: one that runs
// out sets the status word, the CTA stops issuing work, waits (bounded) for its copies in
// flight, frees its tensor memory and returns; the others then run out at the barrier too.
//
// Memory written by one phase (generic stores) is read by the next phase's TMA loads (the
// async proxy) in OTHER CTAs: writers fence the proxy before they arrive at the barrier, the
// TMA thread fences after it has seen the barrier.
#include <stdlib.h>

#include "gemm_tc_kernel.cuh"

#define CH_MAX_PHASES 8
#define CH_MAX_MAPS 8
#define CH_SPIN_LIMIT (1u << 22)
enum { CH_PRODUCT = 0, CH_NORM = 1 };

struct ChPhase {
    int type;
    // product
    TcParams g;
    int mode, map_w, map_a;
    // norm: out[r] = norm(x[rows ? rows[r] : r])
    const float* x;
    const float* w;
    float eps, offset;
    void* nout;
    int nout_bf16;
    const int* rows;
    int n_rows, hidden;
};
struct ChParams {
    int n_phases, n_maps;
    int* barrier;
    int* status;
    ChPhase ph[CH_MAX_PHASES];
};
struct ChMaps {
    CUtensorMap m[CH_MAX_MAPS];
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int atom_add_release_gpu(int* p, int v) {
    int old;
    asm volatile("atom.add.release.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// The K blocks of every product of the chain, in the order this CTA works through them.
struct ChCursor {
    int ph = -1;
    TcSchedule s;
    int tile = 0, kb = 0, kb1 = 0;
    bool have = false;
    __device__ __forceinline__ bool next(const ChParams& cp, int& o_ph, int& o_tile, int& o_kb) {
        for (;;) {
            if (have && kb < kb1) {
                o_ph = ph;
                o_tile = tile;
                o_kb = kb++;
                return true;
            }
            have = false;
            if (ph >= 0 && ph < cp.n_phases && cp.ph[ph].type == CH_PRODUCT && s.next(tile, kb, kb1)) {
                have = true;
                continue;
            }
            if (++ph >= cp.n_phases) return false;
            if (cp.ph[ph].type == CH_PRODUCT) s.init(cp.ph[ph].g);
        }
    }
};

// The epilogue of one work item (tile, K blocks [kb0, kb1)) of a product with epilogue MODE:
// the non-cluster path of gemm_tc_kernel.  Returns false when a wait ran out.
template <int BN, int MODE>
__device__ __forceinline__ void chain_epilogue(const TcParams& p, const TcSchedule& sched, int tile, int kb0, int kb1,
                                               uint32_t lane_addr, uint32_t acce, uint8_t* xchg, int* last_flag, int q, int row,
                                               int et) {
    constexpr int FEAT = MODE == TC_SWIGLU_BF16 ? 64 : TC_BM;
    const int m0 = 0, n0 = tile * FEAT;                 // one token tile: tiles_m == 1
    const bool whole = kb0 == 0 && kb1 == p.kb_total;
    bool finish = whole;
    int contributors = 1;
    constexpr int NV = BN / 4;
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
    if (!whole) {
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
        mbar_arrive(acce);                              // the accumulator buffer is free again
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
            const int prev = atomicAdd(p.counters + tile, 1);
            const int last = (prev == contributors - 1) ? 1 : 0;
            if (last) p.counters[tile] = 0;             // ready for the next product
            *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        finish = *last_flag != 0;
        __threadfence();
    }
    if (finish && !whole) {
        const int tw = et >> 5;
        const float4* src4 = reinterpret_cast<const float4*>(p.partials + (size_t)tile * p.max_slots * (size_t)(BN * TC_BM)) + et;
        float4 acc[NV];
#pragma unroll
        for (int i = 0; i < NV; i++) acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
        for (int z = 0; z < contributors; z++) {
            const float4* pz = src4 + (size_t)z * (BN * TC_BM / 4);
            float4 t[NV];
#pragma unroll
            for (int i = 0; i < NV; i++)
                t[i] = (m0 + i * 4 + tw < p.M) ? __ldcg(pz + i * TC_BM) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int i = 0; i < NV; i++) {
                acc[i].x += t[i].x;
                acc[i].y += t[i].y;
                acc[i].z += t[i].z;
                acc[i].w += t[i].w;
            }
        }
        tc_emit_flat<MODE, BN>(p, m0, n0, acc, et, res, have_res);
    } else if (finish) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
            if (m0 + c >= p.M) break;
            float v[16];
            tmem_ld16(lane_addr + c, v);
            tc_emit_chunk<MODE>(p, m0, n0, c, v, xchg, q, row, et);
        }
    }
    if (whole) {
        tc_fence_before();
        mbar_arrive(acce);
    }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_chain_kernel(const __grid_constant__ ChMaps maps, const __grid_constant__ ChParams cp) {
    constexpr int W_BYTES = TC_BM * TC_BK * 2, A_BYTES = BN * TC_BK * 2, STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 128;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* xchg = smem + STAGES * STAGE_BYTES;
    uint64_t* bars = (uint64_t*)(xchg + TC_XCHG_BYTES);                  // full[S], empty[S], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 4);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* last_flag = (int*)(tmem_slot + 2);
    float* red = (float*)(tmem_slot + 4);                                // [4] warp sums of a norm

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grid = gridDim.x;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES);
    const uint32_t accf0 = smem_u32(bars + 2 * STAGES), acce0 = smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        for (int i = 0; i < cp.n_maps; i++) tma_prefetch_map(&maps.m[i]);
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(accf0 + 8 * b, 1);
            mbar_init(acce0 + 8 * b, 128);
        }
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA thread
        // Two cursors over the same sequence of K blocks: the weight tile of a block is requested
        // as soon as its stage is free, whatever phase it belongs to; its activation tile once the
        // phase that writes the activations has passed the grid barrier.
        if (lane == 0) {
            ChCursor cw, ca;
            int wph = 0, wtile = 0, wkb = 0, aph = 0, atile = 0, akb = 0;
            bool w_more = cw.next(cp, wph, wtile, wkb), a_more = ca.next(cp, aph, atile, akb);
            int gw = 0, ga = 0;               // blocks whose weight / activation tile has been requested
            int done_phases = 0;              // phases known to have passed the barrier
            bool waited = false, alive = true;
            uint32_t idle = 0;
            while ((w_more || a_more) && alive) {
                bool progressed = false;
                if (w_more) {
                    const int s = gw % STAGES;
                    if (mbar_try_wait(empty0 + 8 * s, ((gw / STAGES) & 1) ^ 1)) {
                        const TcParams& p = cp.ph[wph].g;
                        const uint32_t stage = smem_base + s * STAGE_BYTES;
                        mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
                        int x, y;
                        if (cp.ph[wph].mode == TC_SWIGLU_BF16) {
                            tc_w_coords(p, wtile * 64, wkb, x, y);
                            tma_load_2d(stage, &maps.m[cp.ph[wph].map_w], full0 + 8 * s, x, y);
                            tc_w_coords(p, p.up_row0 + wtile * 64, wkb, x, y);
                            tma_load_2d(stage + W_BYTES / 2, &maps.m[cp.ph[wph].map_w], full0 + 8 * s, x, y);
                        } else {
                            tc_w_coords(p, wtile * TC_BM, wkb, x, y);
                            tma_load_2d(stage, &maps.m[cp.ph[wph].map_w], full0 + 8 * s, x, y);
                        }
                        gw++;
                        w_more = cw.next(cp, wph, wtile, wkb);
                        progressed = true;
                    }
                }
                if (!waited && (gw >= STAGES || !w_more)) {
                    pdl_wait();               // what the kernels in front wrote may be read from here on
                    waited = true;
                    progressed = true;
                }
                if (a_more && ga < gw && waited) {
                    if (aph > done_phases) {
                        done_phases = ld_acquire_gpu(cp.barrier) / grid;
                        if (aph <= done_phases) fence_proxy_async_global();
                    }
                    if (aph <= done_phases) {
                        const int s = ga % STAGES;
                        tma_load_2d(smem_base + s * STAGE_BYTES + W_BYTES, &maps.m[cp.ph[aph].map_a], full0 + 8 * s, akb * TC_BK, 0);
                        ga++;
                        a_more = ca.next(cp, aph, atile, akb);
                        progressed = true;
                    }
                }
                if (progressed) {
                    idle = 0;
                } else if (++idle > CH_SPIN_LIMIT || *abort_flag) {
                    if (!*abort_flag) atomicExch(cp.status, 31);
                    *abort_flag = 1;
                    alive = false;
                }
            }
            if (!waited) pdl_wait();
            // copies in flight must land before the CTA may exit
            for (int i = max(0, ga - STAGES); i < ga; i++)
                if (!mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1)) atomicExch(cp.status, 32);
            if (gw > ga) {
                // gave up with weight tiles requested whose stage can never complete (no activation
                // tile): give those copies time to land
                const long long t0 = clock64();
                while (clock64() - t0 < 400000) {}
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA thread
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            const uint64_t desc0 = smem_desc_sw128(smem_base);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            constexpr uint32_t STAGE_STEP = STAGE_BYTES >> 4, A_OFF = W_BYTES >> 4;
            int s = 0, item = 0;
            uint32_t ph = 0;
            bool alive = true;
            TcSchedule sched;
            int tile, kb0, kb1;
            for (int phase = 0; phase < cp.n_phases && alive; phase++) {
                if (cp.ph[phase].type != CH_PRODUCT) continue;
                sched.init(cp.ph[phase].g);
                while (alive && sched.next(tile, kb0, kb1)) {
                    const int buf = item & 1;
                    if (!mbar_wait(acce0 + 8 * buf, ((item >> 1) & 1) ^ 1)) {
                        atomicExch(cp.status, 35);
                        *abort_flag = 1;
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t acc_addr = tmem_base + buf * BN;
                    for (int kb = kb0; kb < kb1; kb++) {
                        if (!mbar_wait(full0 + 8 * s, ph)) {
                            atomicExch(cp.status, 33);
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
                            umma_bf16(acc_addr, wdesc, tdesc, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
                        }
                        umma_commit(empty0 + 8 * s);
                        if (++s == STAGES) { s = 0; ph ^= 1; }
                    }
                    if (!alive) break;
                    umma_commit(accf0 + 8 * buf);
                    item++;
                }
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue and norms
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int et = (warp - 2) * 32 + lane;     // 0..127
        pdl_wait();                                // outputs, scratch, counters and the barrier belong to earlier kernels until now
        int item = 0;
        TcSchedule sched;
        int tile, kb0, kb1;
        bool alive = true;
        for (int phase = 0; phase < cp.n_phases && alive; phase++) {
            const ChPhase& P = cp.ph[phase];
            if (P.type == CH_PRODUCT) {
                sched.init(P.g);
                while (sched.next(tile, kb0, kb1)) {
                    const int buf = item & 1;
                    if (!mbar_wait(accf0 + 8 * buf, (item >> 1) & 1)) {
                        atomicExch(cp.status, 34);
                        *abort_flag = 1;
                    }
                    if (*abort_flag) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
                    const uint32_t acce = acce0 + 8 * buf;
                    switch (P.mode) {
                        case TC_STORE_BF16: chain_epilogue<BN, TC_STORE_BF16>(P.g, sched, tile, kb0, kb1, lane_addr, acce, xchg, last_flag, q, row, et); break;
                        case TC_STORE_F32: chain_epilogue<BN, TC_STORE_F32>(P.g, sched, tile, kb0, kb1, lane_addr, acce, xchg, last_flag, q, row, et); break;
                        case TC_ADD_F32: chain_epilogue<BN, TC_ADD_F32>(P.g, sched, tile, kb0, kb1, lane_addr, acce, xchg, last_flag, q, row, et); break;
                        default: chain_epilogue<BN, TC_SWIGLU_BF16>(P.g, sched, tile, kb0, kb1, lane_addr, acce, xchg, last_flag, q, row, et); break;
                    }
                    item++;
                }
            } else {
                // RMSNorm: CTA r takes row r (sum of squares and scaling in float32; the row is read
                // from L2, where the phase before left it)
                const int n4 = P.hidden >> 2;
                const float4* w4 = reinterpret_cast<const float4*>(P.w);
                for (int r = blockIdx.x; r < P.n_rows; r += grid) {
                    const int src = P.rows ? P.rows[r] : r;
                    const float4* x4 = reinterpret_cast<const float4*>(P.x + (size_t)src * P.hidden);
                    float ss = 0.0f;
                    for (int i = et; i < n4; i += 128) {
                        const float4 v = __ldcg(x4 + i);
                        ss = fmaf(v.x, v.x, ss);
                        ss = fmaf(v.y, v.y, ss);
                        ss = fmaf(v.z, v.z, ss);
                        ss = fmaf(v.w, v.w, ss);
                    }
                    ss = warp_sum(ss);
                    if (lane == 0) red[q] = ss;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const float total = ((red[2] + red[3]) + red[0]) + red[1];      // warps 2, 3, 4, 5 in order (q = warp & 3)
                    const float inv = 1.0f / sqrtf(total / (float)P.hidden + P.eps);
                    for (int i = et; i < n4; i += 128) {
                        const float4 v = __ldcg(x4 + i), g = w4[i];
                        const float a = v.x * inv * (P.offset + g.x), b = v.y * inv * (P.offset + g.y);
                        const float c = v.z * inv * (P.offset + g.z), d = v.w * inv * (P.offset + g.w);
                        if (P.nout_bf16) {
                            uint2 pk;
                            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
                            pk.x = *reinterpret_cast<uint32_t*>(&lo);
                            pk.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(P.nout) + (size_t)r * P.hidden + 4 * i) = pk;
                        } else {
                            *reinterpret_cast<float4*>(reinterpret_cast<float*>(P.nout) + (size_t)r * P.hidden + 4 * i) = make_float4(a, b, c, d);
                        }
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");      // `red` is free for the next row
                }
            }
            if (!alive) break;
            // ---- the grid barrier behind the phase: this CTA's stores are fenced (also against
            // TMA reads elsewhere), one thread arrives and waits for everybody
            fence_proxy_async_global();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (et == 0) {
                __threadfence();
                const int old = atom_add_release_gpu(cp.barrier, 1);
                if (phase + 1 < cp.n_phases) {
                    const int target = (phase + 1) * grid;
                    bool ok = old + 1 >= target;
                    for (uint32_t i = 0; !ok && i < CH_SPIN_LIMIT; i++) ok = ld_acquire_gpu(cp.barrier) >= target || *abort_flag;
                    if (!ok) {
                        atomicExch(cp.status, 36);
                        *abort_flag = 1;
                    }
                } else if (old + 1 == cp.n_phases * grid) {
                    *cp.barrier = 0;           // the last arrival of the launch: ready for the next one
                }
                __threadfence();
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*abort_flag) alive = false;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------- host
static int chain_sm_count() {
    static int count[HB_MAX_DEVICES] = {};
    int& n = count[hb_device_slot()];
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    }
    return n;
}

template <int BN, int STAGES>
struct ChLaunch {
    static constexpr int SMEM = STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + TC_XCHG_BYTES + (2 * STAGES + 4) * 8 + 64 + 1024;
    static_assert(SMEM <= 227 * 1024, "the chain's tile pipeline does not fit shared memory");
    // CTAs of this kernel that can be resident at once on the current device (0: the query failed)
    static int resident() {
        static int cached[HB_MAX_DEVICES] = {};
        int& n = cached[hb_device_slot()];
        if (n == 0) {
            if (cudaFuncSetAttribute(gemm_chain_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
                cudaGetLastError();
                n = -1;
            } else {
                int per_sm = 0;
                if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_chain_kernel<BN, STAGES>, TC_THREADS, SMEM) != cudaSuccess) {
                    cudaGetLastError();
                    per_sm = 0;
                }
                n = per_sm > 0 ? per_sm * chain_sm_count() : -1;
            }
        }
        return n > 0 ? n : 0;
    }
    static int launch(const ChMaps& maps, const ChParams& cp, int grid, cudaStream_t s) {
        // the runtime would let a grid that cannot be resident at once wait at its barrier: refuse it here
        if (resident() < grid) return hb_fail("gemm_chain: %d CTAs cannot be resident at once (%d can)", grid, resident());
        cudaError_t e = hb_launch(gemm_chain_kernel<BN, STAGES>, dim3(grid), dim3(TC_THREADS), SMEM, s, maps, cp);
        if (e != cudaSuccess) return hb_fail("gemm_chain: launch failed: %s", cudaGetErrorString(e));
        return hb_check_launch("gemm_chain");
    }
};

static int chain_token_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : 64; }

// Work split of one product of a chain on `grid` CTAs (one token tile).
static void chain_plan(int bn, int N, int K, int mode, int grid, TcParams& p, long long& scratch_floats, long long& tiles) {
    const int feat = mode == TC_SWIGLU_BF16 ? 64 : TC_BM;
    p.tiles_m = 1;
    p.tiles_n = (N + feat - 1) / feat;
    p.kb_total = (K + TC_BK - 1) / TC_BK;
    p.split = 1;
    p.cluster = 0;
    tiles = p.tiles_n;
    const long long kbt = p.kb_total;
    if (tiles >= grid) {
        p.stream_k = 3;
        const long long cut = tiles % grid, base = cut * kbt / grid;
        p.max_slots = base > 0 ? (int)(kbt / base) + 2 : (int)kbt;
        if (p.max_slots > grid) p.max_slots = grid;
        scratch_floats = cut * p.max_slots * (long long)bn * TC_BM;
    } else {
        p.stream_k = 1;
        const long long base = tiles * kbt / grid;
        p.max_slots = base > 0 ? (int)(kbt / base) + 2 : (int)kbt;
        if (p.max_slots > grid) p.max_slots = grid;
        scratch_floats = tiles * p.max_slots * (long long)bn * TC_BM;
    }
}

static int chain_grid(int bn) {
    const int sms = chain_sm_count();
    int res = bn == 16 ? ChLaunch<16, 11>::resident() : bn == 32 ? ChLaunch<32, 10>::resident() : ChLaunch<64, 8>::resident();
    return res < sms ? res : sms;
}

extern "C" int hb_gemm_chain_max_ops(void) { return CH_MAX_PHASES; }
extern "C" int hb_gemm_chain_max_rows(void) { return 64; }

// Scratch the chain needs: float32 partial tiles (the largest need of its products; a grid
// barrier separates them) and one counter per output tile.
extern "C" int hb_gemm_chain_scratch(const HbChainOp* ops, int n_ops, long long* floats, long long* counters) {
    *floats = 0;
    *counters = 0;
    int rows = 1;
    for (int i = 0; i < n_ops; i++) rows = ops[i].type == CH_PRODUCT ? (ops[i].M > rows ? ops[i].M : rows) : (ops[i].n_rows > rows ? ops[i].n_rows : rows);
    HB_REQUIRE(rows <= 64, "gemm_chain: %d rows are more than a chain takes (64)", rows);
    const int bn = chain_token_tile(rows), grid = chain_grid(bn);
    HB_REQUIRE(grid > 0, "gemm_chain: the kernel cannot be resident on this device");
    for (int i = 0; i < n_ops; i++) {
        if (ops[i].type != CH_PRODUCT) continue;
        TcParams p;
        long long f, t;
        chain_plan(bn, ops[i].N, ops[i].K, ops[i].mode, grid, p, f, t);
        if (f > *floats) *floats = f;
        if (t > *counters) *counters = t;
    }
    return 0;
}

// Runs the operations in order, as one launch.  Products: out[M, N] (op)= a[M, K] w[N, K]^T with
// the epilogue `mode` of hb_gemm_tc (and its operand rules); norms: hb_rmsnorm with a hidden
// size that is a multiple of 4 and 16-byte aligned rows.  `barrier` is one int, zero before
// the first use (the kernel leaves it zero); `status` the status words.
extern "C" int hb_gemm_chain(const HbChainOp* ops, int n_ops, float* partials, long long partials_capacity, int* counters,
                             long long counters_capacity, int* barrier, int* status, void* stream) {
    if (n_ops == 0) return 0;
    HB_REQUIRE(n_ops > 0 && n_ops <= CH_MAX_PHASES, "gemm_chain: %d operations (at most %d)", n_ops, CH_MAX_PHASES);
    HB_REQUIRE(barrier != nullptr && status != nullptr, "gemm_chain: no barrier or status word");
    int rows = 1;
    for (int i = 0; i < n_ops; i++) {
        const int r = ops[i].type == CH_PRODUCT ? ops[i].M : ops[i].n_rows;
        HB_REQUIRE(r >= 1 && r <= 64, "gemm_chain: operation %d has %d rows (1 to 64)", i, r);
        if (r > rows) rows = r;
    }
    const int bn = chain_token_tile(rows), grid = chain_grid(bn);
    HB_REQUIRE(grid > 0, "gemm_chain: the kernel cannot be resident on this device");
    ChMaps maps;
    ChParams cp;
    memset(&maps, 0, sizeof maps);
    memset(&cp, 0, sizeof cp);
    cp.n_phases = n_ops;
    cp.barrier = barrier;
    cp.status = status;
    int n_maps = 0;
    for (int i = 0; i < n_ops; i++) {
        const HbChainOp& o = ops[i];
        ChPhase& P = cp.ph[i];
        if (o.type == CH_PRODUCT) {
            P.type = CH_PRODUCT;
            HB_REQUIRE(o.N > 0 && o.K > 0, "gemm_chain: bad sizes N=%d K=%d", o.N, o.K);
            HB_REQUIRE(o.mode >= 0 && o.mode <= 3, "gemm_chain: unknown epilogue %d", o.mode);
            HB_REQUIRE(((uintptr_t)o.a & 15) == 0 && ((uintptr_t)o.w & 15) == 0, "gemm_chain: operands must be 16-byte aligned");
            HB_REQUIRE(o.lda % 8 == 0 && (o.packed || o.ldw % 8 == 0), "gemm_chain: row strides must be multiples of 8 elements");
            HB_REQUIRE(o.lda >= o.K && (o.packed || o.ldw >= o.K) && o.ldc >= o.N, "gemm_chain: a row stride is smaller than its row");
            HB_REQUIRE(!o.packed || o.N <= o.w_rows, "gemm_chain: %d output features from a packed matrix of %lld rows", o.N, o.w_rows);
            HB_REQUIRE(o.mode != TC_SWIGLU_BF16 || (o.up_row0 + o.N <= o.w_rows && (!o.packed || o.up_row0 % 64 == 0)),
                       "gemm_chain: up rows lie outside the weight matrix");
            HB_REQUIRE(o.mode != TC_SWIGLU_BF16 || (o.ldc % 8 == 0 && ((uintptr_t)o.out & 15) == 0),
                       "gemm_chain: the SwiGLU output needs 16-byte aligned rows");
            HB_REQUIRE(n_maps + 2 <= CH_MAX_MAPS, "gemm_chain: more than %d products", CH_MAX_MAPS / 2);
            long long f, t;
            chain_plan(bn, o.N, o.K, o.mode, grid, P.g, f, t);
            HB_REQUIRE(partials && counters && partials_capacity >= f && counters_capacity >= t,
                       "gemm_chain: operation %d needs %lld scratch floats and %lld counters", i, f, t);
            P.g.out = o.out;
            P.g.ldc = o.ldc;
            P.g.M = o.M;
            P.g.N = o.N;
            P.g.K = o.K;
            P.g.up_row0 = o.up_row0;
            P.g.partials = partials;
            P.g.counters = counters;
            P.g.error_flag = status;
            P.g.packed = o.packed ? 1 : 0;
            P.mode = o.mode;
            P.map_w = n_maps;
            P.map_a = n_maps + 1;
            if (tc_make_weight_map(&maps.m[n_maps], o.w, o.w_rows, o.K, o.ldw, o.mode == TC_SWIGLU_BF16 ? 64 : TC_BM, o.packed)) return 1;
            if (tc_make_map(&maps.m[n_maps + 1], o.a, o.M, o.K, o.lda, bn)) return 1;
            n_maps += 2;
        } else if (o.type == CH_NORM) {
            P.type = CH_NORM;
            HB_REQUIRE(o.hidden > 0 && o.hidden % 4 == 0, "gemm_chain: a norm's hidden size %d must be a multiple of 4", o.hidden);
            HB_REQUIRE(((uintptr_t)o.x & 15) == 0 && ((uintptr_t)o.weight & 15) == 0 && ((uintptr_t)o.nout & 15) == 0,
                       "gemm_chain: a norm's rows must be 16-byte aligned");
            HB_REQUIRE(o.out_dtype == HB_BF16 || o.out_dtype == HB_F32, "gemm_chain: a norm writes bfloat16 or float32");
            P.x = o.x;
            P.w = o.weight;
            P.eps = o.eps;
            P.offset = o.offset;
            P.nout = o.nout;
            P.nout_bf16 = o.out_dtype == HB_BF16 ? 1 : 0;
            P.rows = o.rows;
            P.n_rows = o.n_rows;
            P.hidden = o.hidden;
        } else {
            return hb_fail("gemm_chain: unknown operation type %d", o.type);
        }
    }
    cp.n_maps = n_maps;
    cudaStream_t s = (cudaStream_t)stream;
    switch (bn) {
        case 16: return ChLaunch<16, 11>::launch(maps, cp, grid, s);
        case 32: return ChLaunch<32, 10>::launch(maps, cp, grid, s);
    }
    return ChLaunch<64, 8>::launch(maps, cp, grid, s);
}
