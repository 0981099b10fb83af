// Tensor-core matrix product for sm_100a:  C[M,N] (+)= A[M,K] * W[N,K]^T, bfloat16 in,
// float32 accumulation in tensor memory, fed by TMA.  It replaces the reference's WMMA tile
// kernel and its few-row kernel (cleanroom-transformer/src/cuda_backend.cu:93-177) for
// prefill and for decode alike.
//
// Orientation.  The weight tile is the M operand of the MMA (128 output features on the
// 128 TMEM lanes) and the tokens are its N operand (16..256 columns).  A decode step with a
// handful of tokens therefore streams each weight exactly once through a 128 x 64 tile
// pipeline with an N of 16, and a prefill step uses the same kernel with N = 256.
//
// One CTA = one (token tile, feature tile[, K split]).  192 threads:
//   warp 0     TMA producer: one thread arms full[s] with the stage's byte count and issues
//              the tile loads (cp.async.bulk.tensor, 128-byte swizzle, zero fill outside)
//   warp 1     allocates tensor memory; one thread issues tcgen05.mma (K = 16 per
//              instruction, 4 per 64-wide stage) and commits to empty[s] / accum
//   warps 2-5  epilogue: tcgen05.ld the accumulator (lane = feature, column = token) and
//              store / add to the residual / apply SiLU(gate) * up
// Epilogues: STORE (bf16 or f32), ADD (f32 residual += acc; the reference's fused residual
// add, cuda_backend.cu:130,807), SWIGLU (two accumulators, gate and up rows of the same
// features; the reference's fused decode kernel, cuda_backend.cu:551-559).
//
// Split-K (decode only): grid.z CTAs each reduce a K range into float32 partial tiles in a
// scratch buffer; the last CTA of a tile to finish (a counter per tile) adds the partials in
// split order and runs the epilogue, so the sum order is fixed.
//
// Every wait is bounded: a wait that runs out sets *error_flag, the CTA stops issuing work,
// waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// Requirements (checked on the host, refused with a message otherwise): bfloat16 A and W,
// 16-byte aligned bases, row strides that are multiples of 8 elements.  Any M, N and K.
#include <cuda.h>

#include "api.h"
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
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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

template <int BN, bool DUAL>
struct TcLayout {
    static constexpr int W_BYTES = TC_BM * TC_BK * 2;                 // 16 KB
    static constexpr int A_BYTES = BN * TC_BK * 2;
    static constexpr int STAGE_BYTES = W_BYTES * (DUAL ? 2 : 1) + A_BYTES;
    static constexpr int ACC_COLS = BN * (DUAL ? 2 : 1);
    static constexpr int TMEM_COLS = ACC_COLS <= 32 ? 32 : ACC_COLS <= 64 ? 64 : ACC_COLS <= 128 ? 128 : ACC_COLS <= 256 ? 256 : 512;
};

// ------------------------------------------------------------------------------- kernel
template <int BN, int MODE, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a, void* __restrict__ out,
               long long ldc, int M, int N, int K, int up_row0, float* __restrict__ partials,
               int* __restrict__ tile_counters, int* __restrict__ error_flag) {
    constexpr bool DUAL = MODE == TC_SWIGLU_BF16;
    using L = TcLayout<BN, DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + STAGES * L::STAGE_BYTES);      // full[S], empty[S], accum
    uint32_t* tmem_slot = (uint32_t*)(bars + 2 * STAGES + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    int* last_flag = (int*)(tmem_slot + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * BN;          // first token of the tile
    const int n0 = blockIdx.y * TC_BM;       // first feature of the tile
    const int splits = gridDim.z, split = blockIdx.z;
    const int kb_total = (K + TC_BK - 1) / TC_BK;
    const int kb_per = (kb_total + splits - 1) / splits;
    const int kb0 = split * kb_per;
    const int kb1 = min(kb_total, kb0 + kb_per);
    const int nkb = max(0, kb1 - kb0);

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + STAGES), accum = smem_u32(bars + 2 * STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), L::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            int armed = 0, s = 0;
            uint32_t ph = 0;
            // The weights are written by no kernel of a step: the first stages' weight tiles are
            // requested before waiting for the kernel in front, whose output is only the
            // activation operand.
            const int early = min(nkb, STAGES);
            for (int i = 0; i < early; i++) {
                const uint32_t stage = smem_base + i * L::STAGE_BYTES;
                const int k = (kb0 + i) * TC_BK;
                mbar_expect_tx(full0 + 8 * i, L::STAGE_BYTES);
                tma_load_2d(stage, &map_w, full0 + 8 * i, k, n0);
                if (DUAL) tma_load_2d(stage + L::W_BYTES, &map_w, full0 + 8 * i, k, up_row0 + n0);
            }
            pdl_wait();
            for (int i = 0; i < early; i++)
                tma_load_2d(smem_base + i * L::STAGE_BYTES + L::W_BYTES * (DUAL ? 2 : 1), &map_a, full0 + 8 * i,
                            (kb0 + i) * TC_BK, m0);
            armed = early;
            if (early == STAGES) ph = 1; else s = early;
            for (int i = early; i < nkb; i++) {
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1)) {
                    atomicExch(error_flag, 1);
                    *abort_flag = 1;
                    break;
                }
                const uint32_t stage = smem_base + s * L::STAGE_BYTES;
                const int k = (kb0 + i) * TC_BK;
                mbar_expect_tx(full0 + 8 * s, L::STAGE_BYTES);
                tma_load_2d(stage, &map_w, full0 + 8 * s, k, n0);
                if (DUAL) tma_load_2d(stage + L::W_BYTES, &map_w, full0 + 8 * s, k, up_row0 + n0);
                tma_load_2d(stage + L::W_BYTES * (DUAL ? 2 : 1), &map_a, full0 + 8 * s, k, m0);
                armed = i + 1;
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            // copies in flight must land before the CTA may exit: wait (bounded) for the
            // stages armed last; a stage the MMA thread already consumed answers at once
            for (int i = max(0, armed - STAGES); i < armed; i++)
                if (!mbar_wait(full0 + 8 * (i % STAGES), (i / STAGES) & 1)) atomicExch(error_flag, 2);
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        // One thread issues every MMA of the tile, so its instruction stream is the critical
        // path for few-token tiles: descriptors are advanced with one 32-bit add per MMA
        // (the high word is constant) and nothing else is recomputed inside the loop.
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16(BN);
            const uint64_t desc0 = smem_desc_sw128(smem_base);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            constexpr uint32_t STAGE_STEP = L::STAGE_BYTES >> 4, A_OFF = (L::W_BYTES * (DUAL ? 2 : 1)) >> 4,
                               UP_OFF = L::W_BYTES >> 4;
            int s = 0;
            uint32_t ph = 0;
            for (int i = 0; i < nkb; i++) {
                if (!mbar_wait(full0 + 8 * s, ph)) {
                    atomicExch(error_flag, 3);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t w_lo = desc_lo0 + s * STAGE_STEP;
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; kk++) {
                    const uint64_t wdesc = ((uint64_t)desc_hi << 32) | (w_lo + 2 * kk);
                    const uint64_t tdesc = ((uint64_t)desc_hi << 32) | (w_lo + A_OFF + 2 * kk);
                    const uint32_t acc = (i | kk) ? 1u : 0u;
                    umma_bf16(tmem_base, wdesc, tdesc, idesc, acc);
                    if (DUAL) umma_bf16(tmem_base + BN, ((uint64_t)desc_hi << 32) | (w_lo + UP_OFF + 2 * kk), tdesc, idesc, acc);
                }
                umma_commit(empty0 + 8 * s);      // frees the stage when these MMAs have read it
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
            umma_commit(accum);                    // arrives when every MMA above has finished
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                    // TMEM lane quarter this warp may read
        const int f = n0 + q * 32 + lane;          // feature of this thread
        bool ok = true;
        pdl_wait();                                // the output, the scratch and the counters belong to earlier kernels until now
        if (!mbar_wait(accum, 0)) {
            atomicExch(error_flag, 4);
            *abort_flag = 1;
            ok = false;
        }
        if (*abort_flag) ok = false;
        tc_fence_after();
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const bool have_acc = nkb > 0;
        if (ok && splits > 1) {
            // partial tile to scratch: [tile][split][token][feature], float32
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
            float* p = partials + (tile * splits + split) * (size_t)(BN * TC_BM);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                float v[16];
                if (have_acc) tmem_ld16(lane_addr + c, v);
#pragma unroll
                for (int j = 0; j < 16; j++) p[(size_t)(c + j) * TC_BM + q * 32 + lane] = have_acc ? v[j] : 0.0f;
            }
            __threadfence();
        }
        // the four epilogue warps agree on who finishes the tile
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (splits > 1) {
            if (threadIdx.x == 64) {
                const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
                const int prev = atomicAdd(tile_counters + tile, 1);
                const int last = (prev == splits - 1) ? 1 : 0;
                if (last) tile_counters[tile] = 0;      // ready for the next launch
                *last_flag = last;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (!*last_flag) ok = false;
            __threadfence();
        }
        if (ok) {
            const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;
                float v[16], u[16];
                if (splits > 1) {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = 0.0f;
                    for (int z = 0; z < splits; z++) {
                        const float* p = partials + (tile * splits + z) * (size_t)(BN * TC_BM);
#pragma unroll
                        for (int j = 0; j < 16; j++) v[j] += __ldcg(p + (size_t)(c + j) * TC_BM + q * 32 + lane);
                    }
                } else if (have_acc) {
                    tmem_ld16(lane_addr + c, v);
                    if (DUAL) tmem_ld16(lane_addr + BN + c, u);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = u[j] = 0.0f;
                }
                if (f < N) {
                    if (MODE == TC_ADD_F32) {
                        // all loads of the residual first, then the stores: written one by one the
                        // compiler must keep each load behind the store before it (they may alias)
                        float r[16];
                        float* po = (float*)out + (size_t)(m0 + c) * ldc + f;
#pragma unroll
                        for (int j = 0; j < 16; j++) r[j] = (m0 + c + j < M) ? __ldcg(po + (size_t)j * ldc) : 0.0f;
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (m0 + c + j < M) po[(size_t)j * ldc] = r[j] + v[j];
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int m = m0 + c + j;
                            if (m < M) {
                                const size_t o = (size_t)m * ldc + f;
                                if (MODE == TC_STORE_BF16) ((bf16*)out)[o] = __float2bfloat16_rn(v[j]);
                                else if (MODE == TC_STORE_F32) ((float*)out)[o] = v[j];
                                else ((bf16*)out)[o] = __float2bfloat16_rn(silu_f32(v[j]) * u[j]);
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Tensor map of a row-major bf16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zeros outside.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return hb_fail("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return hb_fail("gemm_tc: tensor map encode failed with code %d (rows %lld cols %lld ld %lld)", (int)r, rows, cols, ld);
    return 0;
}

template <int BN, int MODE, int STAGES>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& ma, void* out, long long ldc, int M, int N, int K,
                     int up_row0, int splits, float* partials, int* counters, int* error_flag, cudaStream_t s) {
    using L = TcLayout<BN, MODE == TC_SWIGLU_BF16>;
    constexpr int SMEM = STAGES * L::STAGE_BYTES + (2 * STAGES + 1) * 8 + 16 + 1024;
    static_assert(SMEM <= 227 * 1024, "tile pipeline does not fit shared memory");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, MODE, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) return hb_fail("gemm_tc: cannot reserve %d bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
        attr_set = true;
    }
    dim3 grid((M + BN - 1) / BN, (N + TC_BM - 1) / TC_BM, splits);
    hb_launch(gemm_tc_kernel<BN, MODE, STAGES>, dim3(grid), dim3(TC_THREADS), SMEM, s, mw, ma, out, ldc, M, N, K, up_row0, partials, counters, error_flag);
    return hb_check_launch("gemm_tc");
}

template <int MODE>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& ma, void* out, long long ldc, int M, int N, int K,
                       int up_row0, int splits, float* partials, int* counters, int* error_flag, cudaStream_t s) {
    constexpr bool DUAL = MODE == TC_SWIGLU_BF16;
    switch (bn) {
        case 16: return launch_tc<16, MODE, DUAL ? 6 : 12>(mw, ma, out, ldc, M, N, K, up_row0, splits, partials, counters, error_flag, s);
        case 32: return launch_tc<32, MODE, DUAL ? 5 : 8>(mw, ma, out, ldc, M, N, K, up_row0, splits, partials, counters, error_flag, s);
        case 64: return launch_tc<64, MODE, DUAL ? 5 : 8>(mw, ma, out, ldc, M, N, K, up_row0, splits, partials, counters, error_flag, s);
        case 128: return launch_tc<128, MODE, DUAL ? 4 : 6>(mw, ma, out, ldc, M, N, K, up_row0, splits, partials, counters, error_flag, s);
        case 256: return launch_tc<256, MODE, DUAL ? 3 : 4>(mw, ma, out, ldc, M, N, K, up_row0, splits, partials, counters, error_flag, s);
    }
    return hb_fail("gemm_tc: token tile %d is not built", bn);
}

extern "C" int hb_gemm_tc_token_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// Scratch floats that a split-K launch needs: one BN x 128 partial tile per (tile, split).
extern "C" long long hb_gemm_tc_scratch_floats(int M, int N, int splits) {
    if (splits <= 1) return 0;
    const int bn = hb_gemm_tc_token_tile(M);
    const long long tiles = (long long)((M + bn - 1) / bn) * ((N + TC_BM - 1) / TC_BM);
    return tiles * splits * bn * TC_BM;
}

extern "C" long long hb_gemm_tc_tiles(int M, int N) {
    const int bn = hb_gemm_tc_token_tile(M);
    return (long long)((M + bn - 1) / bn) * ((N + TC_BM - 1) / TC_BM);
}

// mode: 0 store bf16, 1 store f32, 2 add into f32, 3 silu(gate) * up -> bf16 (W holds the gate
// rows [0, N) and the up rows [up_row0, up_row0 + N)).  splits > 1 needs `partials`
// (hb_gemm_tc_scratch_floats floats) and `tile_counters` (hb_gemm_tc_tiles ints, zero before the
// first use; the kernel leaves them zero).  `error_flag` is a device int the kernel sets
// when a wait ran out.
extern "C" int hb_gemm_tc(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out,
                          long long ldc, int M, int N, int K, int mode, int up_row0, int splits, float* partials,
                          int* tile_counters, int* error_flag, void* stream) {
    if (M == 0 || N == 0) return 0;
    HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    HB_REQUIRE(mode >= 0 && mode <= 3, "gemm_tc: unknown epilogue %d", mode);
    HB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    HB_REQUIRE(lda % 8 == 0 && ldw % 8 == 0, "gemm_tc: row strides %lld and %lld must be multiples of 8 elements", lda, ldw);
    HB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_tc: a row stride is smaller than its row");
    HB_REQUIRE(error_flag != nullptr, "gemm_tc: no error flag");
    HB_REQUIRE(splits >= 1 && splits <= 32, "gemm_tc: %d K splits", splits);
    HB_REQUIRE(splits == 1 || (partials && tile_counters && mode != TC_SWIGLU_BF16), "gemm_tc: split-K needs scratch and no SwiGLU");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 + N <= w_rows, "gemm_tc: up rows lie outside the weight matrix");
    const int bn = hb_gemm_tc_token_tile(M);
    CUtensorMap mw, ma;
    if (make_map(&mw, w, w_rows, K, ldw, TC_BM)) return 1;
    if (make_map(&ma, a, M, K, lda, bn)) return 1;
    cudaStream_t s = (cudaStream_t)stream;
    switch (mode) {
        case TC_STORE_BF16: return dispatch_bn<TC_STORE_BF16>(bn, mw, ma, out, ldc, M, N, K, up_row0, splits, partials, tile_counters, error_flag, s);
        case TC_STORE_F32: return dispatch_bn<TC_STORE_F32>(bn, mw, ma, out, ldc, M, N, K, up_row0, splits, partials, tile_counters, error_flag, s);
        case TC_ADD_F32: return dispatch_bn<TC_ADD_F32>(bn, mw, ma, out, ldc, M, N, K, up_row0, splits, partials, tile_counters, error_flag, s);
        default: return dispatch_bn<TC_SWIGLU_BF16>(bn, mw, ma, out, ldc, M, N, K, up_row0, splits, partials, tile_counters, error_flag, s);
    }
}
