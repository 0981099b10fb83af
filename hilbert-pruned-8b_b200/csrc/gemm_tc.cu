// Tensor-core matrix product for sm_100a:  C[M,N] (+)= A[M,K] * W[N,K]^T, bfloat16 in,
// float32 accumulation in tensor memory, fed by TMA.  It replaces the reference's WMMA tile
// kernel and its few-row kernel (cleanroom-transformer/src/cuda_backend.cu:93-177) for
// prefill and for decode alike.
//
// Orientation.  The weight tile is the M operand of the MMA (128 weight rows on the 128 TMEM
// lanes) and the tokens are its N operand (16..256 columns).  A decode step with a handful
// of tokens streams each weight exactly once through a 128 x 64 tile pipeline with an N of
// 16; a prefill step uses the same kernel with N = 256.
//
// Persistent CTAs (one per SM), 192 threads each:
//   warp 0     TMA producer: one thread arms full[s] with the stage's byte count and issues
//              the tile loads (cp.async.bulk.tensor, 128-byte swizzle, zero fill outside);
//              it runs ahead across work items, so the pipeline never drains between tiles
//   warp 1     allocates tensor memory; one thread issues tcgen05.mma (K = 16 per
//              instruction, 4 per 64-wide stage) into one of two accumulator buffers and
//              commits to empty[s] / acc_full[buffer]
//   warps 2-5  epilogue: tcgen05.ld the accumulator (lane = weight row, column = token),
//              write the result, hand the buffer back (acc_empty) -- while the MMA thread
//              already fills the other buffer with the next work item
// Epilogues: STORE (bf16 or f32), ADD (f32 residual += acc; the reference's fused residual
// add, cuda_backend.cu:130,807), SWIGLU (the tile's 128 weight rows are 64 gate rows and
// the 64 up rows of the same features; the epilogue pairs lanes i and i + 64 through shared
// memory; the reference's fused decode kernel, cuda_backend.cu:551-559).
//
// Work split.  Many-token products: output tiles round-robin over the CTAs.  Few-token
// products (one token tile, decode): stream-K -- the (tile, K block) space is cut into one
// contiguous range per CTA, so every SM streams the same number of weight bytes; a CTA that
// holds only part of a tile's K range writes a float32 partial tile to scratch, and the last
// contributor of a tile (a counter per tile) adds the partials in K order and runs the
// epilogue, so the sum order is fixed.
//
// Every wait is bounded: a wait that runs out sets *error_flag, the CTA stops issuing work,
// waits (bounded) for its own copies in flight, frees its tensor memory and returns.
//
// Requirements (checked on the host, refused with a message otherwise): bfloat16 A and W,
// 16-byte aligned bases, row strides that are multiples of 8 elements.  Any M, N and K.
#include <stdlib.h>

#include "gemm_tc_kernel.cuh"

// ------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// Tensor map of a row-major bf16 matrix [rows, cols] with row stride ld (elements): boxes of
// box_rows x 64 elements, 128-byte swizzle, zeros outside.
int tc_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
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

int tc_make_out_map(CUtensorMap* map, const void* base, int elem_bytes, long long rows, long long cols, long long ld,
                    int box_rows, int box_cols) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return hb_fail("gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return hb_fail("gemm_tc: output tensor map encode failed with code %d (rows %lld cols %lld ld %lld)", (int)r, rows, cols, ld);
    return 0;
}

// The map of a weight matrix: row-major [rows, K] with row stride ld, or packed tiles, which
// read as a matrix of 64-column rows (ceil(rows / 128) * ceil(K / 64) * 128 of them).
int tc_make_weight_map(CUtensorMap* map, const void* w, long long rows, long long K, long long ld, int box_rows, int packed) {
    if (!packed) return tc_make_map(map, w, rows, K, ld, box_rows);
    const long long bands = (rows + TC_BM - 1) / TC_BM, kbs = (K + TC_BK - 1) / TC_BK;
    return tc_make_map(map, w, bands * kbs * TC_BM, TC_BK, TC_BK, box_rows);
}

static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        if (n <= 0) n = 1;
    }
    return n;
}

extern "C" int hb_gemm_tc_token_tile(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

static bool clusters_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("HILBERT_B200_CLUSTER");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// The work split of a product: tiles, grid, stream-K or not, scratch.  schedule: 0 automatic,
// 1 whole tiles round-robin, 2 stream-K, 3 cut tiles first and whole tiles after.
struct TcPlan {
    int bn, feat, tiles_m, tiles_n, kb_total, grid, stream_k, max_slots, split, cluster;
    long long scratch_floats, tiles;
};
// whether `tiles` clusters of `size` CTAs of the cluster variant for token tile `bn` can be
// resident at once, and whether `size` partial tiles fit over its pipeline stages
static bool clusters_fit_mode(int bn, int mode, int size, long long tiles);

static TcPlan make_plan(int M, int N, int K, int mode, int schedule) {
    TcPlan pl;
    pl.bn = hb_gemm_tc_token_tile(M);
    pl.feat = mode == TC_SWIGLU_BF16 ? 64 : TC_BM;
    pl.tiles_m = (M + pl.bn - 1) / pl.bn;
    pl.tiles_n = (N + pl.feat - 1) / pl.feat;
    pl.tiles = (long long)pl.tiles_m * pl.tiles_n;
    pl.kb_total = (K + TC_BK - 1) / TC_BK;
    const int sms = sm_count();
    const long long units = pl.tiles * pl.kb_total;
    // Few tiles: K is cut.  Tiles enough to fill the device run whole when there are several
    // token tiles, or when the token tile is above 64: its partial tiles (64 KB and more) cost
    // more than the last wave's idle SMs (gate/up product of 128 tokens: 65-74 us cut, 61 us whole).
    const bool few = pl.tiles < sm_count();
    pl.stream_k = schedule == 2 || (schedule == 0 && (few || (pl.tiles_m == 1 && pl.bn <= 64)));
    pl.split = 1;
    pl.cluster = 0;
    if (schedule == 3 || (schedule == 0 && pl.stream_k && pl.tiles >= sms)) {
        // As many tiles as SMs or more: tiles % SMs tiles are cut over all CTAs first, then
        // every CTA takes tiles / SMs whole tiles: the sums of the cut tiles overlap the whole
        // tiles and the kernel ends with plain epilogues.
        pl.stream_k = 3;
        pl.grid = (int)(units < sms ? units : sms);
        const long long cut_tiles = pl.tiles % pl.grid, base = cut_tiles * pl.kb_total / pl.grid;
        pl.max_slots = base > 0 ? (int)(pl.kb_total / base) + 2 : pl.kb_total;
        if (pl.max_slots > pl.grid) pl.max_slots = pl.grid;
        pl.scratch_floats = cut_tiles * pl.max_slots * (long long)pl.bn * TC_BM;
    } else if (pl.stream_k) {
        // Few tiles: either every SM takes one contiguous range of the whole (tile, K block)
        // space, or each tile is cut into floor(SMs / tiles) equal K ranges (one work item per
        // CTA, fewer partial tiles).  Costs in K blocks; a work item costs about six K blocks
        // of fixed time (partial tile, counter, reduction).
        long long g = units / 4;                  // at least four K blocks per CTA
        g = g < 1 ? 1 : g > sms ? sms : g;
        if (schedule == 0 && pl.tiles < sms) {
            long long split = sms / pl.tiles;
            // The K ranges of a tile as one cluster, which sums in shared memory (fixed time of
            // about four K blocks instead of six), if all clusters can be resident at once;
            // up to a fifth fewer ranges than SMs allow are accepted for that.  (Fewer, longer
            // ranges look better when one product is timed alone, 9.7 against 11.6 us for 64
            // tokens x 2048 x 2048 in clusters of 4 instead of 128 ranges; inside a step they
            // lose 1-4 %: with a range per SM the whole matrix is requested before the kernel in
            // front has finished.)
            bool cluster = false;
            if (pl.bn <= 64 && clusters_enabled())
                for (long long s = split < TC_MAX_CLUSTER ? split : TC_MAX_CLUSTER; s >= 2 && s * 5 >= split * 4; s--)
                    if (pl.kb_total / s >= 4 && clusters_fit_mode(pl.bn, mode, (int)s, pl.tiles)) {
                        split = s;
                        cluster = true;
                        break;
                    }
            const long long aligned_cost = (pl.kb_total + split - 1) / split + (cluster ? 4 : 6);
            const long long stream_cost = units / g + 12;
            if (aligned_cost <= stream_cost && pl.kb_total / split >= 4) {
                pl.stream_k = 2;
                pl.split = (int)split;
                pl.cluster = cluster ? 1 : 0;
                g = pl.tiles * split;
            }
        }
        pl.grid = (int)g;
        const long long base = units / pl.grid;
        pl.max_slots = pl.stream_k == 2 ? pl.split : (int)(pl.kb_total / base) + 2;
        if (pl.max_slots > pl.grid) pl.max_slots = pl.grid;
        pl.scratch_floats = pl.tiles * pl.max_slots * (long long)pl.bn * TC_BM;
    } else {
        pl.grid = (int)(pl.tiles < sms ? pl.tiles : sms);
        pl.max_slots = 0;
        pl.scratch_floats = 0;
    }
    return pl;
}

// Scratch a product needs: float32 partial tiles (hb_gemm_tc_scratch_floats) and one int
// counter per output tile (hb_gemm_tc_tiles; zero before the first use, the kernel leaves
// them zero).
extern "C" long long hb_gemm_tc_scratch_floats(int M, int N, int K, int mode, int schedule) {
    return make_plan(M, N, K, mode, schedule).scratch_floats;
}
extern "C" long long hb_gemm_tc_tiles(int M, int N, int mode) { return make_plan(M, N, 64, mode, 1).tiles; }

// How many clusters of `size` CTAs of the 16-token cluster variant can be resident at once
// (diagnostics and tests; 0 if the size is not built).
extern "C" int hb_gemm_tc_resident_clusters(int mode, int size) {
    if (size < 2 || size > TC_MAX_CLUSTER) return 0;
    switch (mode & 3) {
        case TC_STORE_BF16: return TcClusterLaunch<16, TC_STORE_BF16>::resident_clusters(size);
        case TC_STORE_F32: return TcClusterLaunch<16, TC_STORE_F32>::resident_clusters(size);
        case TC_ADD_F32: return TcClusterLaunch<16, TC_ADD_F32>::resident_clusters(size);
        default: return TcClusterLaunch<16, TC_SWIGLU_BF16>::resident_clusters(size);
    }
}

static bool clusters_fit_mode(int bn, int mode, int size, long long tiles) {
    switch (bn) {
        case 16: return clusters_fit_bn<16>(mode, size, tiles);
        case 32: return clusters_fit_bn<32>(mode, size, tiles);
        case 64: return tc_wide_clusters_fit(bn, mode, size, tiles);
    }
    return false;
}

static int dispatch_bn(int bn, bool cluster, int mode, const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid,
                       cudaStream_t s) {
    switch (bn) {
        case 16: return tc_launch_bn<16, 11>(cluster, mode, mw, ma, prm, grid, s);
        case 32: return tc_launch_bn<32, 10>(cluster, mode, mw, ma, prm, grid, s);
    }
    return tc_wide_launch(bn, cluster, mode, mw, ma, prm, grid, s);
}

// mode: 0 store bf16, 1 store f32, 2 add into f32, 3 silu(gate) * up -> bf16 (W holds the gate
// rows [0, N) and the up rows [up_row0, up_row0 + N); up_row0 = -1: W holds them in bands of 128
// rows, the gate rows of features 64 b .. 64 b + 63 followed by their up rows, which a tile
// reads as one box instead of two).  `partials` and `tile_counters` are the
// scratch described above (capacities in floats and ints); `error_flag` is a device int the
// kernel sets when a wait ran out.  `packed`: W is stored as contiguous 128 x 64 tiles (see
// tc_w_coords; w_rows is then the number of rows before padding and ldw is not used).
//
// `fold` (may be null): a norm between two products folded into them, for up to TC_SCALE_ROWS
// tokens.  The product that writes the residual stream (mode 2) also writes bf16(x * (offset +
// weight)) and per token the sums of squares of each 32 features; the product that reads it
// (modes 0, 1, 3) multiplies every token's row by rsqrt(sum * inv_size + eps).
extern "C" int hb_gemm_tc_fold(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out,
                               long long ldc, int M, int N, int K, int mode, int up_row0, int schedule, float* partials,
                               long long partials_capacity, int* tile_counters, long long counters_capacity, int* error_flag,
                               int packed, const HbNormFold* fold, void* stream) {
    if (M == 0 || N == 0) return 0;
    HB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    HB_REQUIRE(mode >= 0 && mode <= 3, "gemm_tc: unknown epilogue %d", mode);
    HB_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    HB_REQUIRE(lda % 8 == 0 && (packed || ldw % 8 == 0), "gemm_tc: row strides %lld and %lld must be multiples of 8 elements", lda, ldw);
    HB_REQUIRE(lda >= K && (packed || ldw >= K) && ldc >= N, "gemm_tc: a row stride is smaller than its row");
    HB_REQUIRE(!packed || N <= w_rows, "gemm_tc: %d output features from a packed matrix of %lld rows", N, w_rows);
    HB_REQUIRE(!packed || mode != TC_SWIGLU_BF16 || up_row0 % 64 == 0 || up_row0 == -1, "gemm_tc: packed up rows must start at a multiple of 64");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 >= -1, "gemm_tc: up rows start at %d", up_row0);
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 != -1 || (N % 64 == 0 && 2LL * N <= w_rows),
               "gemm_tc: [gate; up] in bands needs a multiple of 64 features and both halves in the matrix");
    HB_REQUIRE(error_flag != nullptr, "gemm_tc: no error flag");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || up_row0 < 0 || up_row0 + N <= w_rows, "gemm_tc: up rows lie outside the weight matrix");
    HB_REQUIRE(mode != TC_SWIGLU_BF16 || (ldc % 8 == 0 && ((uintptr_t)out & 15) == 0),
               "gemm_tc: the SwiGLU output needs 16-byte aligned rows");
    const TcPlan pl = make_plan(M, N, K, mode, schedule);
    if (pl.stream_k) {
        HB_REQUIRE(partials && tile_counters && partials_capacity >= pl.scratch_floats && counters_capacity >= pl.tiles,
                   "gemm_tc: stream-K needs %lld scratch floats and %lld counters", pl.scratch_floats, pl.tiles);
    }
    CUtensorMap mw, ma;
    if (tc_make_weight_map(&mw, w, w_rows, K, ldw, mode == TC_SWIGLU_BF16 && up_row0 >= 0 ? 64 : TC_BM, packed)) return 1;
    if (tc_make_map(&ma, a, M, K, lda, pl.bn)) return 1;
    TcParams prm = {};
    if (fold != nullptr && fold->prep_w != nullptr) {
        HB_REQUIRE(mode == TC_ADD_F32 && M <= TC_SCALE_ROWS && pl.tiles_m == 1, "gemm_tc: a norm is prepared by the product that adds to the residual, for up to %d tokens", TC_SCALE_ROWS);
        HB_REQUIRE(N % 4 == 0 && ldc % 4 == 0 && ((uintptr_t)out & 15) == 0, "gemm_tc: preparing a norm needs 16-byte aligned output rows");
        HB_REQUIRE(fold->prep_out != nullptr && fold->prep_sumsq != nullptr && ((uintptr_t)fold->prep_out & 7) == 0 && fold->prep_ld % 4 == 0 &&
                       fold->prep_ld >= N && ((uintptr_t)fold->prep_w & 15) == 0,
                   "gemm_tc: the prepared norm input needs 8-byte aligned rows of at least %d elements", N);
        HB_REQUIRE(fold->sumsq_ld >= (N + 31) / 32, "gemm_tc: %d sums of squares per token do not fit rows of %d", (N + 31) / 32, fold->sumsq_ld);
        prm.prep_w = fold->prep_w;
        prm.prep_offset = fold->prep_offset;
        prm.prep_out = (bf16*)fold->prep_out;
        prm.prep_ld = fold->prep_ld;
        prm.prep_sumsq = fold->prep_sumsq;
        prm.sumsq_ld = fold->sumsq_ld;
    }
    if (fold != nullptr && fold->scale_sumsq != nullptr) {
        HB_REQUIRE(mode != TC_ADD_F32 && M <= TC_SCALE_ROWS && pl.tiles_m == 1, "gemm_tc: rows are scaled for up to %d tokens, not in the residual add", TC_SCALE_ROWS);
        HB_REQUIRE(fold->scale_parts > 0 && fold->scale_parts <= fold->sumsq_ld && fold->sumsq_ld % 4 == 0 && ((uintptr_t)fold->scale_sumsq & 15) == 0,
                   "gemm_tc: %d sums of squares per token in rows of %d floats", fold->scale_parts, fold->sumsq_ld);
        prm.scale_sumsq = fold->scale_sumsq;
        prm.scale_parts = fold->scale_parts;
        prm.scale_inv_size = fold->scale_inv_size;
        prm.scale_eps = fold->scale_eps;
        prm.sumsq_ld = fold->sumsq_ld;
    }
    prm.out = out;
    prm.ldc = ldc;
    prm.M = M;
    prm.N = N;
    prm.K = K;
    prm.up_row0 = up_row0;
    prm.tiles_m = pl.tiles_m;
    prm.tiles_n = pl.tiles_n;
    prm.kb_total = pl.kb_total;
    prm.stream_k = pl.stream_k;
    prm.split = pl.split;
    prm.max_slots = pl.max_slots;
    prm.partials = partials;
    prm.counters = tile_counters;
    prm.error_flag = error_flag;
    prm.packed = packed ? 1 : 0;
    const bool cluster = pl.cluster != 0;      // the K ranges of a tile are one cluster (make_plan)
    prm.cluster = cluster ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    return dispatch_bn(pl.bn, cluster, mode, mw, ma, prm, pl.grid, s);
}

extern "C" int hb_gemm_tc(const void* a, long long lda, const void* w, long long ldw, long long w_rows, void* out,
                          long long ldc, int M, int N, int K, int mode, int up_row0, int schedule, float* partials,
                          long long partials_capacity, int* tile_counters, long long counters_capacity, int* error_flag,
                          int packed, void* stream) {
    return hb_gemm_tc_fold(a, lda, w, ldw, w_rows, out, ldc, M, N, K, mode, up_row0, schedule, partials, partials_capacity, tile_counters,
                           counters_capacity, error_flag, packed, nullptr, stream);
}
