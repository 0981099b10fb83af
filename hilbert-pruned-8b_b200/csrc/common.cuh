// Shared device helpers and the host-side error convention of the kernel library.
//
// Every exported function returns 0 on success; on failure it returns non-zero and the
// message is available from hb_last_error() (the reference's set_error/last_error pair,
// cleanroom-transformer/src/base.c:13-21).  Nothing here aborts, traps or allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define HB_PAGE_TOKENS 64

enum HbDtype { HB_F32 = 0, HB_BF16 = 1 };

int hb_fail(const char* fmt, ...);
int hb_check_launch(const char* what);

#define HB_REQUIRE(cond, ...)                \
    do {                                     \
        if (!(cond)) return hb_fail(__VA_ARGS__); \
    } while (0)

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  Every kernel of the library is launched with the
// "programmatic stream serialization" attribute, so it may be scheduled while the kernel
// before it in the stream is still running; it calls pdl_wait() before it touches anything
// that kernel may have written (for most kernels: first thing) and pdl_trigger() to let the
// kernel after it be scheduled early in turn.  What runs before pdl_wait() may only read
// memory that no kernel of a step writes (weights) and set up on-chip state.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool hb_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = hb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max for blocks of up to 1024 threads; every thread gets the result.
// `scratch` is shared memory of at least 33 floats.  The order of the additions is fixed
// by the thread layout, so the result does not depend on what else runs.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float r = lane < nwarp ? scratch[lane] : 0.0f;
        r = warp_sum(r);
        if (lane == 0) scratch[32] = r;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float r = lane < nwarp ? scratch[lane] : -INFINITY;
        r = warp_max(r);
        if (lane == 0) scratch[32] = r;
    }
    __syncthreads();
    return scratch[32];
}

// silu(z) = z / (1 + exp(-z))  (cleanroom-transformer/src/ops_common.h:56)
__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }

// Address of token position `pos` of kv head `g` in a paged cache layer
// [pages][kv_heads][HB_PAGE_TOKENS][head_dim]; `page` is the physical page.
__device__ __forceinline__ size_t cache_offset(int page, int g, int pos, int nkv, int hd) {
    return (((size_t)page * nkv + g) * HB_PAGE_TOKENS + (pos & (HB_PAGE_TOKENS - 1))) * (size_t)hd;
}
