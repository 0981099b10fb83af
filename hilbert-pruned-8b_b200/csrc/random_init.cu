// Random weights on the device: every element a function of (stream base, element index).
//
// The reference has no random-weights mode in its engine (its tests draw checkpoints in
// PyTorch, cleanroom-transformer/tools/parity.py:58-69); this is the library's own.  The CPU
// restatement (weights/random_init.py) gives the same bits: the hash is integer arithmetic,
// and every floating operation below is a single correctly rounded 32-bit add, multiply,
// divide or square root (the _rn intrinsics are never contracted into fused multiply-adds);
// no library logarithm or cosine is called, because those round differently on a CPU.
//
//   z = mix64(base + (i + 1) * G)             the SplitMix64 sequence from `base`
//   p = (float(z >> 32) + 0.5) * 2^-33        a probability in (0, 1/2]
//   x = +-quantile(p)                         Acklam's rational approximation; bit 0 of z is the sign
//   out[i] = mean + std * x                   rounded to nearest-even for bfloat16
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
// one Horner step, two roundings
__device__ __forceinline__ float step(float acc, float x, float c) { return add(mul(acc, x), c); }

// log of a positive normal number: p = m * 2^e with m in [sqrt(1/2), sqrt(2)),
// log m = 2 atanh((m - 1) / (m + 1)) by its series up to the ninth power
__device__ __forceinline__ float log32(float p) {
    const unsigned bits = __float_as_uint(p);
    int e = (int)(bits >> 23) - 126;
    float m = __uint_as_float((bits & 0x007FFFFFu) | 0x3F000000u);      // [0.5, 1)
    if (m < 0x1.6a09e6p-1f) {
        m = mul(m, 2.0f);
        e -= 1;
    }
    const float t = __fdiv_rn(add(m, -1.0f), add(m, 1.0f));
    const float t2 = mul(t, t);
    float s = step(t2, 0x1.c71c72p-4f, 0x1.24924ap-3f);               // t2 / 9 + 1 / 7
    s = step(s, t2, 0x1.99999ap-3f);
    s = step(s, t2, 0x1.555556p-2f);
    s = step(s, t2, 1.0f);
    return add(mul(mul(2.0f, t), s), mul(__int2float_rn(e), 0x1.62e43p-1f));
}

__device__ __forceinline__ float standard_normal(unsigned long long base, unsigned long long i) {
    const unsigned long long z = mix64(base + (i + 1ull) * 0x9E3779B97F4A7C15ULL);
    const float p = mul(add(__uint2float_rn((unsigned)(z >> 32)), 0.5f), 0x1p-33f);
    float x;
    if (p < 0x1.8d4fep-6f) {                                           // 0.02425: the tail
        const float q = __fsqrt_rn(mul(-2.0f, log32(p)));
        float num = -0x1.fe30dap-8f;
        num = step(num, q, -0x1.4a224cp-2f);
        num = step(num, q, -0x1.334c0cp+1f);
        num = step(num, q, -0x1.465da2p+1f);
        num = step(num, q, 0x1.17fa8p+2f);
        num = step(num, q, 0x1.7815c2p+1f);
        float den = 0x1.fe2d86p-8f;
        den = step(den, q, 0x1.4a34d2p-2f);
        den = step(den, q, 0x1.38fa28p+1f);
        den = step(den, q, 0x1.e09076p+1f);
        x = __fdiv_rn(num, step(den, q, 1.0f));
    } else {
        const float q = add(p, -0.5f);
        const float r = mul(q, q);
        float num = -0x1.3d931cp+5f;
        num = step(num, r, 0x1.b9e468p+7f);
        num = step(num, r, -0x1.13edb2p+8f);
        num = step(num, r, 0x1.14b72cp+7f);
        num = step(num, r, -0x1.eaa304p+4f);
        num = step(num, r, 0x1.40d932p+1f);
        float den = -0x1.b3cf0cp+5f;
        den = step(den, r, 0x1.432bf2p+7f);
        den = step(den, r, -0x1.3765ep+7f);
        den = step(den, r, 0x1.0b348cp+6f);
        den = step(den, r, -0x1.a8fb58p+3f);
        x = __fdiv_rn(mul(num, q), step(den, r, 1.0f));
    }
    return (z & 1ull) ? x : -x;
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, unsigned long long n, unsigned long long base, float stdev,
                                     float mean) {
    pdl_trigger();
    pdl_wait();
    const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = from_f32<T>(add(mul(standard_normal(base, i), stdev), mean));
}

}  // namespace

// out[i] = mean + stdev * N(0, 1) for the stream `base` (weights/random_init.py: stream_base)
extern "C" int hb_random_normal(void* out, int out_dtype, long long n, unsigned long long base, float stdev, float mean,
                                void* stream) {
    HB_REQUIRE(n >= 0, "random_normal: negative element count");
    HB_REQUIRE(out_dtype == HB_F32 || out_dtype == HB_BF16, "random_normal: output must be float32 or bfloat16");
    if (n == 0) return 0;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    cudaError_t e;
    if (out_dtype == HB_BF16)
        e = hb_launch(random_normal_kernel<bf16>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (bf16*)out,
                      (unsigned long long)n, base, stdev, mean);
    else
        e = hb_launch(random_normal_kernel<float>, dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, (float*)out,
                      (unsigned long long)n, base, stdev, mean);
    if (e != cudaSuccess) return hb_fail("random_normal: launch failed: %s", cudaGetErrorString(e));
    return hb_check_launch("random_normal");
}
