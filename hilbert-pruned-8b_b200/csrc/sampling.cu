// Sampling on the device: greedy (largest logit, lowest index on ties) and temperature
// sampling by inverse CDF.  The reference samples nothing (it reads option logits and
// takes a softmax over them, cleanroom-transformer/src/engine.c:8-14); both samplers are
// this library's own.
//
// Temperature sampling: p = softmax(logits / T) in float32; a uniform u in [0,1) is derived
// from (seed, request id, step) by a 64-bit mixing function, so a request's draw does not
// depend on what else is in the batch; the token is the first index whose cumulative
// probability exceeds u.  Rows whose temperature is <= 0 are taken greedily.
#include "api.h"
#include "common.cuh"

#define SM_THREADS 1024

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

// 24-bit uniform in [0, 1) from (seed, request, step)
__device__ __forceinline__ float uniform_from(long long seed, long long request, long long step) {
    unsigned long long z = (unsigned long long)seed * 0x9E3779B97F4A7C15ULL +
                           (unsigned long long)request * 0xBF58476D1CE4E5B9ULL +
                           (unsigned long long)step * 0x94D049BB133111EBULL + 0x2545F4914F6CDD1DULL;
    z = mix64(mix64(z));
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Also reports (to every thread) whether the row holds a value that is not finite.
__device__ __forceinline__ void argmax_row(const float* __restrict__ row, int vocab, int* out_idx, float* out_max,
                                           float* sval, int* sidx, bool* out_nonfinite) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    bool bad = false;                      // x - x is 0 for a finite x, NaN for an infinity or a NaN
    if ((((uintptr_t)row) & 15) == 0) {
        // 16-byte loads, four in flight per thread: one block has to pull a whole row
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = vocab >> 2;
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * blockDim.x;
                v[u] = i < n4 ? r4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int base = (i0 + u * blockDim.x) * 4;
                const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    if (i0 + u * blockDim.x < n4) bad |= (e[k] - e[k]) != 0.0f;      // not the padding of a short tail
                    if (e[k] > best || (e[k] == best && base + k < bi)) { best = e[k]; bi = base + k; }
                }
            }
        }
        for (int i = (n4 << 2) + threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            bad |= (v - v) != 0.0f;
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const float v = row[i];
            bad |= (v - v) != 0.0f;
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
    }
    *out_nonfinite = __syncthreads_or(bad ? 1 : 0) != 0;
    // a NaN never compares greater: a row of NaNs yields index 0x7fffffff, mapped to 0 below
    // (a valid token for whatever runs next; the status word tells the host not to use it)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) { sval[warp] = best; sidx[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nwarp ? sval[lane] : -INFINITY;
        bi = lane < nwarp ? sidx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { sval[32] = best; sidx[32] = (bi == 0x7fffffff) ? 0 : bi; }
    }
    __syncthreads();
    *out_idx = sidx[32];
    *out_max = sval[32];
}

// Greedy pick.  A row of a vocabulary-sized logit vector is half a megabyte: one block per row
// leaves most SMs idle for a small batch, so a row is cut into `parts` ranges (grid: parts x
// rows).  Each block leaves (maximum, index) of its range in scratch; the last block of a row to
// finish (a counter per row, left at zero) takes the best of them, lowest index on ties.
__global__ void __launch_bounds__(SM_THREADS)
argmax_kernel(const float* __restrict__ logits, long long stride, int* __restrict__ out, int vocab, int chunk,
              float* part_val, int* part_idx, int* counters, int* status) {
    pdl_trigger();
    pdl_wait();
    logits = pdl_fresh(logits);
    __shared__ float sval[33];
    __shared__ int sidx[33];
    __shared__ int is_last;
    const int part = blockIdx.x, parts = gridDim.x, r = blockIdx.y;
    const int begin = min(part * chunk, vocab), n = min(chunk, vocab - begin);
    int idx = 0;
    float mx = -INFINITY;
    bool nonfinite = false;
    if (n > 0) argmax_row(logits + (size_t)r * stride + begin, n, &idx, &mx, sval, sidx, &nonfinite);
    idx += begin;
    // the reference fails a row whose logits are not finite (engine.c:29-31)
    if (threadIdx.x == 0 && nonfinite) hb_note(status, HB_STATUS_NONFINITE, 1 + r);
    if (parts == 1) {
        if (threadIdx.x == 0) out[r] = idx;
        return;
    }
    if (threadIdx.x == 0) {
        part_val[(size_t)r * parts + part] = n > 0 ? mx : -INFINITY;
        part_idx[(size_t)r * parts + part] = idx;
        __threadfence();
        const int prev = atomicAdd(counters + r, 1);
        is_last = prev == parts - 1;
        if (is_last) counters[r] = 0;                  // ready for the next launch
    }
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        __threadfence();
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int p = 0; p < parts; p++) {              // ranges in index order: the first maximum wins a tie
            const float v = __ldcg(part_val + (size_t)r * parts + p);
            const int i = __ldcg(part_idx + (size_t)r * parts + p);
            if (v > best) { best = v; bi = i; }
        }
        out[r] = bi == 0x7fffffff ? 0 : bi;
    }
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, long long stride, const float* __restrict__ temperature,
              const long long* __restrict__ seeds, const long long* __restrict__ request_ids,
              const long long* __restrict__ steps, int* __restrict__ out, int vocab, int* status) {
    pdl_trigger();
    pdl_wait();
    logits = pdl_fresh(logits);
    __shared__ float sval[33];
    __shared__ int sidx[33];
    __shared__ float prefix[SM_THREADS];
    __shared__ int chosen;
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * stride;
    int amax;
    float mx;
    bool nonfinite;
    argmax_row(row, vocab, &amax, &mx, sval, sidx, &nonfinite);
    if (nonfinite) {                            // engine.c:29-31: such a row is an error, not a draw
        if (tid == 0) {
            out[r] = amax;
            hb_note(status, HB_STATUS_NONFINITE, 1 + r);
        }
        return;
    }
    const float temp = temperature[r];
    if (!(temp > 0.0f)) {
        if (tid == 0) out[r] = amax;
        return;
    }
    const float inv_t = 1.0f / temp;
    // each thread owns a contiguous chunk so that the cumulative sum runs in index order
    const int chunk = (vocab + SM_THREADS - 1) / SM_THREADS;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);
    float part = 0.0f;
    for (int i = begin; i < end; i++) part += expf((row[i] - mx) * inv_t);
    // inclusive scan of the per-thread sums (Hillis-Steele over shared memory)
    prefix[tid] = part;
    __syncthreads();
    for (int o = 1; o < SM_THREADS; o <<= 1) {
        const float add = tid >= o ? prefix[tid - o] : 0.0f;
        __syncthreads();
        prefix[tid] += add;
        __syncthreads();
    }
    const float total = prefix[SM_THREADS - 1];
    const float u = uniform_from(seeds[r], request_ids[r], steps[r]);
    const float target = u * total;
    if (tid == 0) chosen = 0x7fffffff;
    __syncthreads();
    const float incl = prefix[tid], excl = tid > 0 ? prefix[tid - 1] : 0.0f;
    if (begin < end && target >= excl && target < incl) {
        float run = excl;
        int pick = end - 1;
        for (int i = begin; i < end; i++) {
            run += expf((row[i] - mx) * inv_t);
            if (run > target) { pick = i; break; }
        }
        atomicMin(&chosen, pick);
    }
    __syncthreads();
    if (tid == 0) out[r] = (chosen == 0x7fffffff) ? amax : chosen;  // rounding left no interval: the mode
}

// `scratch` (2 * rows * parts 32-bit words) and `counters` (one int per row, zero before the first
// use; left at zero) let a row be cut into `parts` ranges; without them parts is 1.
extern "C" int hb_argmax(const float* logits, long long stride, int* out, int n_rows, int vocab, int parts, void* scratch,
                         int* counters, int* status, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "argmax: bad sizes");
    HB_REQUIRE(n_rows <= 65535, "argmax: too many rows for one launch");
    if (parts < 1 || scratch == nullptr || counters == nullptr) parts = 1;
    int chunk = ((vocab + parts - 1) / parts + 3) & ~3;          // ranges start on 16 bytes when the row does
    parts = (vocab + chunk - 1) / chunk;
    float* part_val = (float*)scratch;
    int* part_idx = (int*)scratch + (size_t)n_rows * parts;
    hb_launch(argmax_kernel, dim3(parts, n_rows), dim3(SM_THREADS), 0, (cudaStream_t)stream, logits, stride, out, vocab, chunk,
              part_val, part_idx, counters, status);
    return hb_check_launch("argmax");
}

extern "C" int hb_sample(const float* logits, long long stride, const float* temperature, const long long* seeds,
                         const long long* request_ids, const long long* steps, int* out, int n_rows, int vocab,
                         int* status, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "sample: bad sizes");
    hb_launch(sample_kernel, dim3(n_rows), dim3(SM_THREADS), 0, (cudaStream_t)stream, logits, stride, temperature, seeds, request_ids,
                                                                   steps, out, vocab, status);
    return hb_check_launch("sample");
}
