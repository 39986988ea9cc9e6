// Host-side launch helper shared by the per-kind instantiation files.
#pragma once
#include "gemm_sm100.cuh"

namespace qgemm {

// Stages per tile width: a stage holds a 128x128-byte A tile and a BNx128-byte B tile.
template <int BN>
struct StagesFor {
    static constexpr int value = (BN == 256) ? 4 : 6;
};

template <int KIND, int BN, int OUT>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
    constexpr int STAGES = StagesFor<BN>::value;
    auto kernel = gemm_tcgen05_kernel<KIND, BN, STAGES, OUT>;
    constexpr int smem = GemmSmem<BN, STAGES>::kDynamicBytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured[dev] = true;
    }
    kernel<<<grid, kGemmThreads, smem, stream>>>(ta, tb, p);
    return cudaGetLastError();
}

template <int KIND>
cudaError_t launch_kind(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                        cudaStream_t stream) {
#define QGEMM_CASE(BN_, OUT_) \
    if (bn == BN_ && out == OUT_) return launch_one<KIND, BN_, OUT_>(ta, tb, p, grid, stream);
    QGEMM_CASE(256, OUT_F32)
    QGEMM_CASE(256, OUT_BF16)
    QGEMM_CASE(256, OUT_F16)
    QGEMM_CASE(256, OUT_RAW32)
    QGEMM_CASE(128, OUT_F32)
    QGEMM_CASE(128, OUT_BF16)
    QGEMM_CASE(128, OUT_F16)
    QGEMM_CASE(128, OUT_RAW32)
#undef QGEMM_CASE
    return cudaErrorInvalidValue;
}

// Defined one per translation unit so the kinds compile in parallel.
cudaError_t launch_gemm_f16(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                            int grid, cudaStream_t stream);
cudaError_t launch_gemm_i8(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                           int grid, cudaStream_t stream);
cudaError_t launch_gemm_f8(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                           int grid, cudaStream_t stream);

}  // namespace qgemm
