// General-shape matrix product  C[M,N] (+)= A[M,K] * W[N,K]^T  on the FP32 pipes.
//
// This is the true 32-bit path of every projection (FFMA, float32 accumulation in a fixed
// order along K), and the fallback of the bfloat16 path for shapes the tensor-core kernel
// refuses.  Inputs may be float32 or bfloat16 in any mix; they are widened exactly.  The
// reference's counterparts are its general fallback and few-row kernels
// (cleanroom-transformer/src/cuda_backend.cu:138-207); `accumulate` is its fused residual
// add (cuda_backend.cu:130,807).
//
// Tile: 64 x 64 outputs per block of 256 threads, K in steps of 16, 4 x 4 outputs per thread.
// Each output is a single chain of fused multiply-adds over K = 0..K-1, so a row's result
// does not depend on which other rows share the call.
#include "api.h"
#include "common.cuh"

#define GB_M 64
#define GB_N 64
#define GB_K 16

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_general_kernel(const TA* __restrict__ A, long long lda, const TW* __restrict__ W, long long ldw,
                    TO* __restrict__ C, long long ldc, int M, int N, int K, int accumulate) {
    pdl_trigger();
    pdl_wait();
    A = pdl_fresh(A);
    __shared__ float As[GB_K][GB_M + 4];
    __shared__ float Ws[GB_K][GB_N + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;       // 16 x 16 threads; thread owns rows ty*4.., cols tx*4..
    const int m0 = blockIdx.y * GB_M, n0 = blockIdx.x * GB_N;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    // each thread loads 4 elements of A and 4 of W per K step: row = tid / 4, k = (tid % 4) * 4 ..
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += GB_K) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int k = k0 + lk + e;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + e][lr] = (am < M && k < K) ? to_f32(A[(size_t)am * lda + k]) : 0.0f;
            Ws[lk + e][lr] = (wn < N && k < K) ? to_f32(W[(size_t)wn * ldw + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GB_K; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            TO* p = C + (size_t)m * ldc + n;
            float v = acc[i][j];
            if (accumulate) v += to_f32(*p);
            *p = from_f32<TO>(v);
        }
    }
}

template <typename TA, typename TW>
static int launch_out(const void* a, long long lda, const void* w, long long ldw, void* out, int out_dtype,
                      long long ldc, int M, int N, int K, int accumulate, cudaStream_t s) {
    dim3 grid((N + GB_N - 1) / GB_N, (M + GB_M - 1) / GB_M);
    if (grid.y > 65535) return hb_fail("gemm_general: %d rows are too many for one call", M);
    if (out_dtype == HB_F32)
        hb_launch(gemm_general_kernel<TA, TW, float>, dim3(grid), dim3(256), 0, s, (const TA*)a, lda, (const TW*)w, ldw, (float*)out, ldc, M,
                                                                 N, K, accumulate);
    else if (out_dtype == HB_BF16)
        hb_launch(gemm_general_kernel<TA, TW, bf16>, dim3(grid), dim3(256), 0, s, (const TA*)a, lda, (const TW*)w, ldw, (bf16*)out, ldc, M, N,
                                                                K, accumulate);
    else
        return hb_fail("gemm_general: unsupported output dtype %d", out_dtype);
    return hb_check_launch("gemm_general");
}

extern "C" int hb_gemm_general(const void* a, int a_dtype, long long lda, const void* w, int w_dtype, long long ldw,
                               void* out, int out_dtype, long long ldc, int M, int N, int K, int accumulate,
                               void* stream) {
    if (M == 0 || N == 0) return 0;
    HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_general: bad sizes M=%d N=%d K=%d", M, N, K);
    HB_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_general: a row stride is smaller than its row");
    cudaStream_t s = (cudaStream_t)stream;
    if (a_dtype == HB_F32 && w_dtype == HB_F32) return launch_out<float, float>(a, lda, w, ldw, out, out_dtype, ldc, M, N, K, accumulate, s);
    if (a_dtype == HB_BF16 && w_dtype == HB_BF16) return launch_out<bf16, bf16>(a, lda, w, ldw, out, out_dtype, ldc, M, N, K, accumulate, s);
    if (a_dtype == HB_F32 && w_dtype == HB_BF16) return launch_out<float, bf16>(a, lda, w, ldw, out, out_dtype, ldc, M, N, K, accumulate, s);
    if (a_dtype == HB_BF16 && w_dtype == HB_F32) return launch_out<bf16, float>(a, lda, w, ldw, out, out_dtype, ldc, M, N, K, accumulate, s);
    return hb_fail("gemm_general: unsupported input dtypes %d x %d", a_dtype, w_dtype);
}
