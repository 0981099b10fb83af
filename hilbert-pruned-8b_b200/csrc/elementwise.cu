// Embedding gather, RMSNorm, SiLU-multiply, rotary table and rotary + cache append.
//
// General-shape kernels: any hidden width, head size and head count.  Formulas follow the
// reference (file:line cited per kernel, paths within cleanroom-transformer/src/).
#include "api.h"
#include "common.cuh"

// ---------------------------------------------------------------------------------- embed
// x[t,:] = float(E[token[t],:])   (cpu_backend.c:236; cuda_backend.cu:66-70)
// `kbt` > 0: the table is stored as the tensor-core products store a weight (contiguous tiles
// of 128 rows x 64 columns, the tiles of a 128-row band one after another along the columns,
// kbt of them): a tied output head and the embedding then share ONE copy of the table.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const TW* __restrict__ table, float* __restrict__ out,
                             int hidden, int vocab, int kbt, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 || tok >= vocab) {         // the host checks what it knows; tokens a sampler left on the device it cannot
        if (threadIdx.x == 0) hb_note(status, HB_STATUS_TOKEN, 1 + t);
        tok = 0;                           // never read outside the table
    }
    float* o = out + (size_t)t * hidden;
    if (kbt > 0) {
        const TW* band = table + ((size_t)(tok >> 7) * kbt * 128 + (tok & 127)) * 64;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(band[(size_t)(i >> 6) * (128 * 64) + (i & 63)]);
    } else {
        const TW* row = table + (size_t)tok * hidden;
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32(row[i]);
    }
}

extern "C" int hb_embed(const int* tokens, const void* table, int table_dtype, float* out, int n_tokens, int hidden,
                        int vocab, int packed, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embed: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int kbt = packed ? (hidden + 63) / 64 : 0;
    if (table_dtype == HB_BF16)
        hb_launch(embed_kernel<bf16>, dim3(n_tokens), dim3(256), 0, s, tokens, (const bf16*)table, out, hidden, vocab, kbt, status);
    else if (table_dtype == HB_F32)
        hb_launch(embed_kernel<float>, dim3(n_tokens), dim3(256), 0, s, tokens, (const float*)table, out, hidden, vocab, kbt, status);
    else
        return hb_fail("embed: unsupported table dtype %d", table_dtype);
    return hb_check_launch("embed");
}

// -------------------------------------------------------------------------------- rmsnorm
// out = x * (1 / sqrt(mean(x^2) + eps)) * (offset + w), sum of squares in float32
// (cpu_backend.c:57-62; cuda_backend.cu:73-85).  Row r of `out` is made from row rows[r]
// of `x` (rows == nullptr: row r).
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, float offset,
                               TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_trigger();
    pdl_wait();
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float* xr = x + (size_t)src * hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = xr[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<TO>(xr[i] * inv * (offset + w[i]));
}

// The same, reading each row once: a thread keeps its 4 * VEC elements in registers between
// the sum of squares and the scaling.  For rows of a multiple of 4 up to 4 * VEC * 256 floats.
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w, float eps, float offset,
                    TO* __restrict__ out, const int* __restrict__ rows, int hidden) {
    pdl_trigger();
    pdl_wait();
    x = pdl_fresh(x);
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * hidden);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const int n4 = hidden >> 2;
    float4 v[VEC];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        const int c = threadIdx.x + i * 256;
        v[i] = c < n4 ? xr[c] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[i].x, v[i].x, ss);
        ss = fmaf(v[i].y, v[i].y, ss);
        ss = fmaf(v[i].z, v[i].z, ss);
        ss = fmaf(v[i].w, v[i].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)hidden + eps);
    TO* o = out + (size_t)r * hidden;
#pragma unroll
    for (int i = 0; i < VEC; i++) {
        const int c = threadIdx.x + i * 256;
        if (c < n4) {
            const float4 g = wr[c];
            const float a = v[i].x * inv * (offset + g.x), b = v[i].y * inv * (offset + g.y);
            const float cc = v[i].z * inv * (offset + g.z), d = v[i].w * inv * (offset + g.w);
            if (sizeof(TO) == 2) {
                uint2 pk;
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(cc, d);
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(o) + 4 * c) = pk;
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + 4 * c) = make_float4(a, b, cc, d);
            }
        }
    }
}

template <typename TO>
static void launch_rmsnorm(const float* x, const float* weight, float eps, float offset, TO* out, const int* rows,
                           int n_rows, int hidden, cudaStream_t s) {
    const bool vec = hidden % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)weight & 15) == 0 &&
                     ((uintptr_t)out & 15) == 0;
    if (vec && hidden <= 4 * 256 * 2)
        hb_launch(rmsnorm_rows_kernel<TO, 2>, dim3(n_rows), dim3(256), 0, s, x, weight, eps, offset, out, rows, hidden);
    else if (vec && hidden <= 4 * 256 * 4)
        hb_launch(rmsnorm_rows_kernel<TO, 4>, dim3(n_rows), dim3(256), 0, s, x, weight, eps, offset, out, rows, hidden);
    else if (vec && hidden <= 4 * 256 * 8)
        hb_launch(rmsnorm_rows_kernel<TO, 8>, dim3(n_rows), dim3(256), 0, s, x, weight, eps, offset, out, rows, hidden);
    else
        hb_launch(rmsnorm_kernel<TO>, dim3(n_rows), dim3(hidden >= 2048 ? 512 : 256), 0, s, x, weight, eps, offset, out, rows,
                  hidden);
}

extern "C" int hb_rmsnorm(const float* x, const float* weight, float eps, float offset, void* out, int out_dtype,
                          const int* rows, int n_rows, int hidden, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && hidden > 0, "rmsnorm: bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == HB_BF16)
        launch_rmsnorm<bf16>(x, weight, eps, offset, (bf16*)out, rows, n_rows, hidden, s);
    else if (out_dtype == HB_F32)
        launch_rmsnorm<float>(x, weight, eps, offset, (float*)out, rows, n_rows, hidden, s);
    else
        return hb_fail("rmsnorm: unsupported output dtype %d", out_dtype);
    return hb_check_launch("rmsnorm");
}

// ------------------------------------------------------------------------------- silu_mul
// out[t,i] = silu(gu[t,i]) * gu[t,inter+i]   (cpu_backend.c:250; cuda_backend.cu:413-416)
template <typename TI, typename TO>
__global__ void silu_mul_kernel(const TI* __restrict__ gu, long long in_stride, TO* __restrict__ out,
                                long long out_stride, int inter) {
    pdl_trigger();
    pdl_wait();
    gu = pdl_fresh(gu);
    const int t = blockIdx.x;
    const int i = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= inter) return;
    const TI* row = gu + (size_t)t * in_stride;
    out[(size_t)t * out_stride + i] = from_f32<TO>(silu_f32(to_f32(row[i])) * to_f32(row[inter + i]));
}

extern "C" int hb_silu_mul(const void* gate_up, int in_dtype, long long in_stride, void* out, int out_dtype,
                           long long out_stride, int n_rows, int inter, void* stream) {
    if (n_rows == 0) return 0;
    HB_REQUIRE(n_rows > 0 && inter > 0, "silu_mul: bad sizes");
    HB_REQUIRE((inter + 255) / 256 <= 65535, "silu_mul: intermediate size %d is too large", inter);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_rows, (inter + 255) / 256);
    if (in_dtype == HB_BF16 && out_dtype == HB_BF16)
        hb_launch(silu_mul_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, s, (const bf16*)gate_up, in_stride, (bf16*)out, out_stride, inter);
    else if (in_dtype == HB_F32 && out_dtype == HB_F32)
        hb_launch(silu_mul_kernel<float, float>, dim3(grid), dim3(256), 0, s, (const float*)gate_up, in_stride, (float*)out, out_stride, inter);
    else if (in_dtype == HB_F32 && out_dtype == HB_BF16)
        hb_launch(silu_mul_kernel<float, bf16>, dim3(grid), dim3(256), 0, s, (const float*)gate_up, in_stride, (bf16*)out, out_stride, inter);
    else
        return hb_fail("silu_mul: unsupported dtypes %d -> %d", in_dtype, out_dtype);
    return hb_check_launch("silu_mul");
}

// ----------------------------------------------------------------------------- rope table
// out[t,i] = (cos, sin)(inv_freq[i] * float(position[t])), the angle a float32 product
// (cpu_backend.c:88-93; cuda_backend.cu:232-236).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ out, int n_tokens, int half) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * half) return;
    const int t = idx / half, i = idx - t * half;
    const float a = __fmul_rn(inv_freq[i], (float)positions[t]);
    float sn, cs;
    sincosf(a, &sn, &cs);
    out[idx] = make_float2(cs, sn);
}

extern "C" int hb_rope_table(const int* positions, const float* inv_freq, float* out, int n_tokens, int half,
                             void* stream) {
    if (n_tokens == 0 || half == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && half > 0, "rope_table: bad sizes");
    const long long n = (long long)n_tokens * half;
    hb_launch(rope_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, (cudaStream_t)stream, positions, inv_freq, (float2*)out,
                                                                                   n_tokens, half);
    return hb_check_launch("rope_table");
}

// --------------------------------------------------------------------- rope + cache append
// Blocks (token, group): a group is ROPE_GROUP query heads, rotated in place, or (the last
// group of a token) all key and value heads: keys are rotated into the cache row of the
// token's position, values are copied there.  Rotation pairs (i, i + rot/2); dims beyond `rot` pass
// through (cpu_backend.c:87-100; cuda_backend.cu:212-249).
#define ROPE_GROUP 8
template <typename T, typename TC>
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(T* __restrict__ qkv, long long qkv_stride, const float2* __restrict__ table, int rot, int nh,
                      int nkv, int hd, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                      const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                      const int* __restrict__ positions, int n_pages, int append, int* status) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int half = rot >> 1;
    // positions and page table are the step's metadata, copied before its first kernel ran:
    // the block that appends looks its page up while the kernel in front still runs
    const bool appends = append && blockIdx.y + 1 == gridDim.y;
    int pos = 0, page = -1;
    if (appends) {
        pos = positions[t];
        page = pos / HB_PAGE_TOKENS < pt_width ? page_table[(size_t)tok_seq[t] * pt_width + pos / HB_PAGE_TOKENS] : -1;
    }
    pdl_wait();
    table = pdl_fresh(table);          // written by the rope table kernel of this step
    T* row = qkv + (size_t)t * qkv_stride;
    const float2* cs_row = table + (size_t)t * half;
    // blockIdx.y < gridDim.y - 1: a group of ROPE_GROUP query heads, rotated in place;
    // the last block of a token handles the key and value heads
    if (!appends) {
        const int h0 = blockIdx.y * ROPE_GROUP, h1 = min(nh, h0 + ROPE_GROUP);
        for (int idx = threadIdx.x; idx < (h1 - h0) * half; idx += blockDim.x) {
            const int h = h0 + idx / half, i = idx % half;
            T* x = row + (size_t)h * hd;
            const float2 cs = cs_row[i];
            float y1, y2;
            rope_pair(to_f32(x[i]), to_f32(x[i + half]), cs.x, cs.y, y1, y2);
            x[i] = from_f32<T>(y1);
            x[i + half] = from_f32<T>(y2);
        }
        return;
    }
    if (page < 0 || page >= n_pages) {         // the host reserved the pages: a fault of its bookkeeping
        if (threadIdx.x == 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
        return;                                // never write outside the cache
    }
    const T* krow = row + (size_t)nh * hd;
    const T* vrow = krow + (size_t)nkv * hd;
    for (int idx = threadIdx.x; idx < nkv * half; idx += blockDim.x) {
        const int g = idx / half, i = idx - g * half;
        const T* x = krow + (size_t)g * hd;
        TC* dst = k_cache + cache_offset(page, g, pos, nkv, hd);
        const float2 cs = cs_row[i];
        float y1, y2;
        rope_pair(to_f32(x[i]), to_f32(x[i + half]), cs.x, cs.y, y1, y2);
        dst[i] = from_f32<TC>(y1);
        dst[i + half] = from_f32<TC>(y2);
    }
    const int tail = hd - rot;
    for (int idx = threadIdx.x; idx < nkv * tail; idx += blockDim.x) {
        const int g = idx / tail, i = rot + idx - g * tail;
        k_cache[cache_offset(page, g, pos, nkv, hd) + i] = from_f32<TC>(to_f32(krow[(size_t)g * hd + i]));
    }
    for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
        const int g = idx / hd, i = idx - g * hd;
        v_cache[cache_offset(page, g, pos, nkv, hd) + i] = from_f32<TC>(to_f32(vrow[idx]));
    }
}

// The same for many bfloat16 tokens: one block per token, 16-byte accesses (8 elements of the
// first half of a head and the matching 8 of the second half per task).  Needs rot % 16 == 0,
// hd % 8 == 0 and 16-byte aligned rows.
__device__ __forceinline__ void rope8(const uint4 lo, const uint4 hi, const float2* __restrict__ cs, uint4& out_lo, uint4& out_hi) {
    const bf16* a = reinterpret_cast<const bf16*>(&lo);
    const bf16* b = reinterpret_cast<const bf16*>(&hi);
    bf16* ya = reinterpret_cast<bf16*>(&out_lo);
    bf16* yb = reinterpret_cast<bf16*>(&out_hi);
#pragma unroll
    for (int e = 0; e < 8; e++) {
        float y1, y2;
        rope_pair(__bfloat162float(a[e]), __bfloat162float(b[e]), cs[e].x, cs[e].y, y1, y2);
        ya[e] = __float2bfloat16_rn(y1);
        yb[e] = __float2bfloat16_rn(y2);
    }
}

__global__ void __launch_bounds__(256)
rope_kv_append_vec_kernel(bf16* __restrict__ qkv, long long qkv_stride, const float2* __restrict__ table, int rot, int nh,
                          int nkv, int hd, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                          const int* __restrict__ page_table, int pt_width, const int* __restrict__ tok_seq,
                          const int* __restrict__ positions, int n_pages, int append, int* status) {
    pdl_trigger();
    pdl_wait();
    table = pdl_fresh(table);
    const int t = blockIdx.x;
    const int half = rot >> 1, hv = half >> 3;                 // 8-element pieces per half head
    bf16* row = qkv + (size_t)t * qkv_stride;
    const float2* cs_row = table + (size_t)t * half;
    int page = -1, pos = 0;
    if (append) {
        pos = positions[t];
        page = pos / HB_PAGE_TOKENS < pt_width ? page_table[(size_t)tok_seq[t] * pt_width + pos / HB_PAGE_TOKENS] : -1;
        if (page < 0 || page >= n_pages) {                     // the host reserved the pages: a fault of its bookkeeping
            if (threadIdx.x == 0) hb_note(status, HB_STATUS_PAGE, 1 + tok_seq[t]);
            page = -1;                                         // never write outside the cache
        }
    }
    const int q_tasks = nh * hv;
    const int k_tasks = page >= 0 ? nkv * hv : 0;
    const int kt_tasks = page >= 0 ? nkv * ((hd - rot) >> 3) : 0;
    const int v_tasks = page >= 0 ? nkv * (hd >> 3) : 0;
    const int total = q_tasks + k_tasks + kt_tasks + v_tasks;
    const bf16* krow = row + (size_t)nh * hd;
    const bf16* vrow = krow + (size_t)nkv * hd;
    for (int task = threadIdx.x; task < total; task += blockDim.x) {
        if (task < q_tasks + k_tasks) {
            const bool is_q = task < q_tasks;
            const int u = is_q ? task : task - q_tasks;
            const int h = u / hv, i = (u - h * hv) << 3;
            const bf16* x = (is_q ? row : krow) + (size_t)h * hd;
            bf16* dst = is_q ? row + (size_t)h * hd : k_cache + cache_offset(page, h, pos, nkv, hd);
            float2 cs[8];
            const float4* c4 = reinterpret_cast<const float4*>(cs_row + i);
#pragma unroll
            for (int e = 0; e < 4; e++) reinterpret_cast<float4*>(cs)[e] = c4[e];
            uint4 o_lo, o_hi;
            rope8(*reinterpret_cast<const uint4*>(x + i), *reinterpret_cast<const uint4*>(x + i + half), cs, o_lo, o_hi);
            *reinterpret_cast<uint4*>(dst + i) = o_lo;
            *reinterpret_cast<uint4*>(dst + i + half) = o_hi;
        } else if (task < q_tasks + k_tasks + kt_tasks) {
            const int u = task - q_tasks - k_tasks, per = (hd - rot) >> 3;
            const int g = u / per, i = rot + ((u - g * per) << 3);
            *reinterpret_cast<uint4*>(k_cache + cache_offset(page, g, pos, nkv, hd) + i) =
                *reinterpret_cast<const uint4*>(krow + (size_t)g * hd + i);
        } else {
            const int u = task - q_tasks - k_tasks - kt_tasks, per = hd >> 3;
            const int g = u / per, i = (u - g * per) << 3;
            *reinterpret_cast<uint4*>(v_cache + cache_offset(page, g, pos, nkv, hd) + i) =
                *reinterpret_cast<const uint4*>(vrow + (size_t)g * hd + i);
        }
    }
}

extern "C" int hb_rope_kv_append(void* qkv, int qkv_dtype, long long qkv_stride, const float* table, int rot,
                                 int n_heads, int n_kv_heads, int head_dim, void* k_cache, void* v_cache,
                                 int cache_dtype, const int* page_table, int pt_width, const int* tok_seq,
                                 const int* positions, int n_tokens, int append, int n_pages, int* status,
                                 void* stream) {
    if (n_tokens == 0) return 0;
    HB_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv_heads > 0 && head_dim > 0, "rope_kv_append: bad sizes");
    HB_REQUIRE(rot >= 0 && rot <= head_dim && rot % 2 == 0, "rope_kv_append: rotary size %d does not fit head size %d",
               rot, head_dim);
    HB_REQUIRE(rot == 0 || table != nullptr, "rope_kv_append: no rotary table");
    if (rot == 0 && !append) return 0;
    const long long work = (long long)ROPE_GROUP * (rot / 2) + (long long)n_kv_heads * head_dim;
    const int threads = work >= 1024 ? 256 : work >= 256 ? 128 : 64;
    const int groups = (n_heads + ROPE_GROUP - 1) / ROPE_GROUP + (append ? 1 : 0);
    HB_REQUIRE(groups <= 65535, "rope_kv_append: too many heads");
    cudaStream_t s = (cudaStream_t)stream;
    const float2* tab = (const float2*)table;
    // many bfloat16 tokens: one block per token with 16-byte accesses (few tokens keep the
    // many small blocks, which finish sooner)
    if (qkv_dtype == HB_BF16 && cache_dtype == HB_BF16 && n_tokens >= 64 && rot > 0 && rot % 16 == 0 && head_dim % 8 == 0 &&
        qkv_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)table & 15) == 0 &&
        ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0) {
        hb_launch(rope_kv_append_vec_kernel, dim3(n_tokens), dim3(256), 0, s, (bf16*)qkv, qkv_stride, tab, rot, n_heads,
                  n_kv_heads, head_dim, (bf16*)k_cache, (bf16*)v_cache, page_table, pt_width, tok_seq, positions, n_pages,
                  append, status);
        return hb_check_launch("rope_kv_append");
    }
    if (qkv_dtype == HB_BF16 && cache_dtype == HB_BF16)
        hb_launch(rope_kv_append_kernel<bf16, bf16>, dim3(n_tokens, groups), dim3(threads), 0, s, (bf16*)qkv, qkv_stride, tab, rot,
                  n_heads, n_kv_heads, head_dim, (bf16*)k_cache, (bf16*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else if (qkv_dtype == HB_F32 && cache_dtype == HB_F32)
        hb_launch(rope_kv_append_kernel<float, float>, dim3(n_tokens, groups), dim3(threads), 0, s, (float*)qkv, qkv_stride, tab, rot,
                  n_heads, n_kv_heads, head_dim, (float*)k_cache, (float*)v_cache, page_table, pt_width, tok_seq, positions,
                  n_pages, append, status);
    else
        return hb_fail("rope_kv_append: unsupported dtypes qkv %d cache %d", qkv_dtype, cache_dtype);
    return hb_check_launch("rope_kv_append");
}
