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

// Device status words: an int32[HB_STATUS_WORDS] of the caller that the host reads where it
// waits anyway.  A kernel that meets a fault traps nothing: it notes the FIRST fault of its
// kind (a non-zero code), carries on with a safe value (a clamped page, a skipped write), and
// the host raises once it has read the words.  A null pointer switches the notes off.
//   [HB_STATUS_WAIT]       a bounded wait of a tensor-core kernel ran out (the code says which)
//   [HB_STATUS_NONFINITE]  a row of logits handed to a sampler was not finite (1 + row)
//   [HB_STATUS_PAGE]       a page number that attention or the cache append needed was outside
//                          the cache, or missing from the page table (1 + sequence's row in the batch)
//   [HB_STATUS_TOKEN]      a token id outside the vocabulary reached the embedding (1 + token's row)
enum { HB_STATUS_WAIT = 0, HB_STATUS_NONFINITE = 1, HB_STATUS_PAGE = 2, HB_STATUS_TOKEN = 3, HB_STATUS_WORDS = 4 };
__device__ __forceinline__ void hb_note(int* status, int word, int code) {
    if (status != nullptr) atomicCAS(status + word, 0, code);
}

// Programmatic dependent launch.  Every kernel of the library is launched with the
// "programmatic stream serialization" attribute, so it may be scheduled while the kernel
// before it in the stream is still running; it calls pdl_wait() before it touches anything
// that kernel may have written (for most kernels: first thing) and pdl_trigger() to let the
// kernel after it be scheduled early in turn.  What runs before pdl_wait() may only read
// memory that no kernel of a step writes (weights) and set up on-chip state.
#ifndef HB_TIMELINE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define TL_INIT()
#define TL_EVENT(code)
#define TL_FLUSH()
#else
// Timeline build (-DHB_TIMELINE): thread 0 of block 0 of every kernel notes the global timer
// when it reaches pdl_wait() (the block is resident and set up) and when the wait returns
// (everything before the kernel in the stream has finished).  The difference between two
// kernels' second marks is the time the first one took inside a replayed graph, overlap
// included.  Each translation unit has its own pointer to the one mark buffer.
static __device__ unsigned long long* g_tl_marks = nullptr;   // [capacity][2]
static __device__ unsigned int* g_tl_count = nullptr;
static __device__ unsigned int g_tl_capacity = 0;
static __device__ int g_tl_events = 0;                        // in-kernel events on (they cost a few microseconds per kernel)
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void pdl_wait() {
    const bool mark = (threadIdx.x | threadIdx.y | blockIdx.x | blockIdx.y | blockIdx.z) == 0 && g_tl_marks != nullptr;
    unsigned long long t0 = 0ull;
    unsigned int i = 0xffffffffu;
    if (mark) {
        t0 = tl_now();
        i = atomicAdd(g_tl_count, 1u);          // the slot is taken while waiting anyway
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (mark && i < g_tl_capacity) {
        g_tl_marks[2 * (size_t)i] = t0;
        g_tl_marks[2 * (size_t)i + 1] = tl_now();
    }
}
// Tagged events inside a kernel: kept in shared memory (a global atomic per event would cost
// the thread a round trip) and copied out by TL_FLUSH at the block's end.  An event is the
// pair (code * 1000 + block, time).
#define TL_EVENTS_PER_BLOCK 128
static __shared__ unsigned long long tl_sh_events[2 * TL_EVENTS_PER_BLOCK];
static __shared__ unsigned int tl_sh_count;
static __shared__ unsigned long long tl_sh_ref[2];      // global timer and SM clock at TL_INIT
static __shared__ int tl_sh_on;                         // the block's copy of g_tl_events
__device__ __forceinline__ void tl_init() {
    tl_sh_count = 0;
    tl_sh_on = g_tl_events;
    if (!tl_sh_on) return;
    tl_sh_ref[0] = tl_now();
    tl_sh_ref[1] = (unsigned long long)clock64();
}
// the SM's cycle counter is cheap to read; the global timer costs a fraction of a microsecond
__device__ __forceinline__ void tl_event(int code) {
    if (!tl_sh_on) return;
    const unsigned long long c = (unsigned long long)clock64();
    const unsigned int i = atomicAdd(&tl_sh_count, 1u);
    if (i < TL_EVENTS_PER_BLOCK) {
        tl_sh_events[2 * i] = (unsigned long long)(code * 1000 + (int)blockIdx.x);
        tl_sh_events[2 * i + 1] = c;
    }
}
__device__ __forceinline__ void tl_flush() {           // the thread that ran tl_init, after a block-wide barrier
    if (!tl_sh_on || g_tl_marks == nullptr) return;
    const unsigned long long g1 = tl_now(), c1 = (unsigned long long)clock64();
    const double ns_per_cycle = (double)(g1 - tl_sh_ref[0]) / (double)(c1 - tl_sh_ref[1]);
    const unsigned int n = min(tl_sh_count, (unsigned int)TL_EVENTS_PER_BLOCK);
    const unsigned int base = atomicAdd(g_tl_count, n);
    for (unsigned int i = 0; i < n && base + i < g_tl_capacity; i++) {
        g_tl_marks[2 * (size_t)(base + i)] = tl_sh_events[2 * i];
        g_tl_marks[2 * (size_t)(base + i) + 1] =
            tl_sh_ref[0] + (unsigned long long)((double)(tl_sh_events[2 * i + 1] - tl_sh_ref[1]) * ns_per_cycle);
    }
}
#ifdef HB_TIMELINE_EVENTS          // a build of its own: the events lengthen the kernels that have them
#define TL_INIT() tl_init()
#define TL_EVENT(code) tl_event(code)
#define TL_FLUSH() tl_flush()
#else
#define TL_INIT()
#define TL_EVENT(code)
#define TL_FLUSH()
#endif
typedef void (*HbTimelineSetter)(unsigned long long*, unsigned int*, unsigned int, int);
void hb_timeline_register(HbTimelineSetter fn);
static void tl_set_this_unit(unsigned long long* marks, unsigned int* count, unsigned int capacity, int events) {
    cudaMemcpyToSymbol(g_tl_events, &events, sizeof events);
    cudaMemcpyToSymbol(g_tl_marks, &marks, sizeof marks);
    cudaMemcpyToSymbol(g_tl_count, &count, sizeof count);
    cudaMemcpyToSymbol(g_tl_capacity, &capacity, sizeof capacity);
}
namespace {
struct TlRegistrar {
    TlRegistrar() { hb_timeline_register(tl_set_this_unit); }
};
static TlRegistrar g_tl_registrar;
}  // namespace
#endif
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// A pointer to memory that an earlier kernel of the step wrote goes through pdl_fresh() after
// pdl_wait().  A plain load through a `const T* __restrict__` parameter counts as a load from
// memory that never changes: the compiler may move it above the wait, whose "memory" clobber
// does not hold it back (seen: a kernel read its queries before the kernel in front had
// written them).  The pointer that comes out of the asm statement carries no such promise.
template <typename T>
__device__ __forceinline__ T* pdl_fresh(T* p) {
    asm volatile("" : "+l"(p)::"memory");
    return p;
}

bool hb_pdl_enabled();

// One-time set-up that belongs to a device (shared-memory opt-ins, SM counts) is kept per
// device: `static bool done[HB_MAX_DEVICES]` indexed by the current device.
#define HB_MAX_DEVICES 64
static inline int hb_device_slot() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= HB_MAX_DEVICES) d = 0;
    return d;
}

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

// The same launch for a kernel that runs as clusters of `cluster_x` CTAs (the size is chosen at
// launch, the kernel carries no __cluster_dims__).
template <typename... KArgs, typename... Args>
static inline cudaError_t hb_launch_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                             unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = hb_pdl_enabled() ? 2 : 1;
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

// One rotated pair (cleanroom-transformer/src/cpu_backend.c:92-97): products rounded to
// float32 one by one, then added, with no fused multiply-add, so that every kernel that
// rotates gives the same bits.
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& y1, float& y2) {
    y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
    y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

// silu(z) = z / (1 + exp(-z))  (cleanroom-transformer/src/ops_common.h:56)
__device__ __forceinline__ float silu_f32(float z) { return z / (1.0f + expf(-z)); }
// The same from the hardware's exp2 and reciprocal (relative error about 2^-21): for results
// that are rounded to bfloat16 at once.  Very negative z gives -0, not NaN: exp2 overflows to +inf and z / inf = -0.
__device__ __forceinline__ float silu_fast(float z) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * z));
    return __fdividef(z, 1.0f + e);
}

// Address of token position `pos` of kv head `g` in a paged cache layer
// [pages][kv_heads][HB_PAGE_TOKENS][head_dim]; `page` is the physical page.
__device__ __forceinline__ size_t cache_offset(int page, int g, int pos, int nkv, int hd) {
    return (((size_t)page * nkv + g) * HB_PAGE_TOKENS + (pos & (HB_PAGE_TOKENS - 1))) * (size_t)hd;
}
