// Token tiles 64, 128 and 256 of the tensor-core matrix product (kernel and scheme: gemm_tc.cu,
// gemm_tc_kernel.cuh): a translation unit of its own, so that the instantiations compile beside
// those of the few-token tiles.
#include "gemm_tc_kernel.cuh"

int tc_wide_launch(int bn, bool cluster, int mode, const CUtensorMap& mw, const CUtensorMap& ma, const TcParams& prm, int grid,
                   cudaStream_t s) {
    switch (bn) {
        case 64: return tc_launch_bn<64, 8>(cluster, mode, mw, ma, prm, grid, s);
        case 128: return tc_launch_bn<128, 6>(cluster, mode, mw, ma, prm, grid, s);
        case 256: return tc_launch_bn<256, 4>(cluster, mode, mw, ma, prm, grid, s);
    }
    return hb_fail("gemm_tc: token tile %d is not built", bn);
}

bool tc_wide_clusters_fit(int bn, int mode, int size, long long tiles) {
    return bn == 64 && clusters_fit_bn<64>(mode, size, tiles);
}
