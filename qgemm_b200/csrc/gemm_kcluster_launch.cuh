// Host-side launch of the in-cluster split-K kernel (gemm_sm100_kcluster.cuh); one translation unit per kind.
#pragma once
#include "gemm_launch.cuh"
#include "gemm_sm100_2cta_kcluster.cuh"
#include "gemm_sm100_kcluster.cuh"

namespace qgemm {

template <int KIND, int BN, int OUT, int AM, int S>
cudaError_t launch_kcluster_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int tiles,
                                cudaStream_t stream) {
    // the kernel has no staging buffers, which leaves room for a seventh stage of the 128-wide tile (the 64-wide
    // tile keeps its even stage count for the two-blocks-per-load grouping)
    // No staging buffers in this kernel, so one more stage fits beside the 128-wide tile's; not with 16 rows of A, where
    // the ring keeps its ten slots for the loads of two K blocks per instruction (an even count).
    constexpr int STAGES = StagesFor<BN, AM>::value + ((BN == 128 && AM != 16) ? 1 : 0);
    auto kernel = gemm_tcgen05_kcluster_kernel<KIND, BN, STAGES, OUT, AM, S>;
    constexpr int smem = GemmSmem<BN, STAGES, AM, true>::kDynamicBytes;
    static_assert(smem <= 227 * 1024, "dynamic shared memory of one CTA");
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles) * S);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, ta, tb, p);
}

// `bn` = tile width (64 or 128), `am` = rows of A loaded per stage (128, or 64 / 32 / 16 for small M),
// `slices` = CTAs per cluster = K slices (2, 4 or 8).
template <int KIND>
cudaError_t launch_kcluster_kind(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                 const GemmParams& p, int tiles, cudaStream_t stream) {
#define QGEMM_KC_CASE(BN_, OUT_, AM_, S_)                          \
    if (bn == BN_ && out == OUT_ && am == AM_ && slices == S_) \
        return launch_kcluster_one<KIND, BN_, OUT_, AM_, S_>(ta, tb, p, tiles, stream);
#define QGEMM_KC_CASES(BN_, AM_, S_)         \
    QGEMM_KC_CASE(BN_, OUT_F32, AM_, S_)     \
    QGEMM_KC_CASE(BN_, OUT_BF16, AM_, S_)    \
    QGEMM_KC_CASE(BN_, OUT_F16, AM_, S_)     \
    QGEMM_KC_CASE(BN_, OUT_RAW32, AM_, S_)
    QGEMM_KC_CASES(128, 128, 2)
    QGEMM_KC_CASES(128, 128, 4)
    QGEMM_KC_CASES(128, 128, 8)
    QGEMM_KC_CASES(128, 64, 2)
    QGEMM_KC_CASES(128, 64, 4)
    QGEMM_KC_CASES(128, 64, 8)
    QGEMM_KC_CASES(128, 32, 2)
    QGEMM_KC_CASES(128, 32, 4)
    QGEMM_KC_CASES(128, 32, 8)
    QGEMM_KC_CASES(128, 16, 2)
    QGEMM_KC_CASES(128, 16, 4)
    QGEMM_KC_CASES(128, 16, 8)
    QGEMM_KC_CASES(64, 128, 2)
    QGEMM_KC_CASES(64, 128, 4)
    QGEMM_KC_CASES(64, 128, 8)
    QGEMM_KC_CASES(64, 64, 2)
    QGEMM_KC_CASES(64, 64, 4)
    QGEMM_KC_CASES(64, 64, 8)
    QGEMM_KC_CASES(64, 32, 2)
    QGEMM_KC_CASES(64, 32, 4)
    QGEMM_KC_CASES(64, 32, 8)
    QGEMM_KC_CASES(64, 16, 2)
    QGEMM_KC_CASES(64, 16, 4)
    QGEMM_KC_CASES(64, 16, 8)
#undef QGEMM_KC_CASES
#undef QGEMM_KC_CASE
    return cudaErrorInvalidValue;
}


// CTA pairs (gemm_sm100_2cta_kcluster.cuh): `tiles` clusters of 2 * `slices` CTAs, one 256 x 128 tile each.
template <int KIND, int OUT, int S>
cudaError_t launch_pair_kcluster_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int tiles,
                                     cudaStream_t stream) {
    auto kernel = gemm_tcgen05_pair_kcluster_kernel<KIND, OUT, S>;
    constexpr int smem = PairSmemT<128, true>::kDynamicBytes;
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(tiles) * 2 * S);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2 * S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, ta, tb, p);
}

template <int KIND>
cudaError_t launch_pair_kcluster_kind(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                      const GemmParams& p, int tiles, cudaStream_t stream) {
#define QGEMM_PKC_CASE(OUT_, S_) \
    if (out == OUT_ && slices == S_) return launch_pair_kcluster_one<KIND, OUT_, S_>(ta, tb, p, tiles, stream);
#define QGEMM_PKC_CASES(S_)       \
    QGEMM_PKC_CASE(OUT_F32, S_)   \
    QGEMM_PKC_CASE(OUT_BF16, S_)  \
    QGEMM_PKC_CASE(OUT_F16, S_)   \
    QGEMM_PKC_CASE(OUT_RAW32, S_)
    QGEMM_PKC_CASES(2)
    QGEMM_PKC_CASES(4)
#undef QGEMM_PKC_CASES
#undef QGEMM_PKC_CASE
    return cudaErrorInvalidValue;
}

}  // namespace qgemm
