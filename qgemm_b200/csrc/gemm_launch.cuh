// Host-side launch helper shared by the per-kind instantiation files.
#pragma once
#include <cstdlib>

#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"
#include "gemm_sm100_2cta_wide.cuh"

namespace qgemm {

// Launch with the programmatic-stream-serialization attribute (see ptx::pdl_wait). QGEMM_PDL=0 in the
// environment turns it off.
inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = std::getenv("QGEMM_PDL");
        v = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Stages per tile width: a stage holds a 128x128-byte A tile and a BNx128-byte B tile.
template <int BN, int AM = kBM>
struct StagesFor {
    // as many as fit in 192 KB, capped at 16
    static constexpr int kFit = (192 * 1024) / ((AM + BN) * 128);
    static constexpr int value = kFit > 16 ? 16 : kFit;
};

// ONE: one tile per CTA (grid == number of tiles): the staging buffers lie over the ring and one more stage fits.
template <int KIND, int BN, int OUT, int AM = kBM, bool ONE = false>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int grid,
                       cudaStream_t stream) {
    constexpr int STAGES = StagesFor<BN, AM>::value + (ONE ? 1 : 0);
    auto kernel = gemm_tcgen05_kernel<KIND, BN, STAGES, OUT, AM, ONE>;
    constexpr int smem = GemmSmem<BN, STAGES, AM, ONE>::kDynamicBytes;
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
    return launch_pdl(kernel, dim3(grid), dim3(kGemmThreads), smem, stream, ta, tb, tc, p);
}

// `am` = rows of A loaded per stage: 128, or 64 / 32 / 16 for small M (64- and 128-wide tiles; 32 / 16 with 256-wide ones). `one` (128-wide tiles, one
// tile per CTA): the layout with a seventh stage.
template <int KIND>
cudaError_t launch_kind(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                        const GemmParams& p, int grid, cudaStream_t stream, bool one = false) {
    if (one && bn == 128 && am == 128) {
        switch (out) {
            case OUT_F32: return launch_one<KIND, 128, OUT_F32, 128, true>(ta, tb, tc, p, grid, stream);
            case OUT_BF16: return launch_one<KIND, 128, OUT_BF16, 128, true>(ta, tb, tc, p, grid, stream);
            case OUT_F16: return launch_one<KIND, 128, OUT_F16, 128, true>(ta, tb, tc, p, grid, stream);
            case OUT_RAW32: return launch_one<KIND, 128, OUT_RAW32, 128, true>(ta, tb, tc, p, grid, stream);
            default: return cudaErrorInvalidValue;
        }
    }
#define QGEMM_CASE(BN_, OUT_, AM_) \
    if (bn == BN_ && out == OUT_ && am == AM_) return launch_one<KIND, BN_, OUT_, AM_>(ta, tb, tc, p, grid, stream);
#define QGEMM_CASES(BN_, AM_)        \
    QGEMM_CASE(BN_, OUT_F32, AM_)   \
    QGEMM_CASE(BN_, OUT_BF16, AM_)  \
    QGEMM_CASE(BN_, OUT_F16, AM_)   \
    QGEMM_CASE(BN_, OUT_RAW32, AM_)
    QGEMM_CASES(256, 128)
    QGEMM_CASES(256, 32)
    QGEMM_CASES(256, 16)
    QGEMM_CASES(128, 128)
    QGEMM_CASES(128, 64)
    QGEMM_CASES(128, 32)
    QGEMM_CASES(128, 16)
    QGEMM_CASES(64, 128)
    QGEMM_CASES(64, 64)
    QGEMM_CASES(64, 32)
    QGEMM_CASES(64, 16)
#undef QGEMM_CASES
#undef QGEMM_CASE
    return cudaErrorInvalidValue;
}

// CTA-pair kernel (256 x 256 tiles, clusters of two); the number of clusters is clamped to what the device can
// keep resident at once (queried once per device). `extra` non-null selects the variant whose epilogue also
// stores every tile to p.n_extra_dst further destinations; `tws` is the tensor map of the last-wave scratch slots
// (read only when p.tail_begin > 0).
template <int KIND, int OUT, bool GATHER, int BN = kPairTileN, bool ONE = false>
cudaError_t launch_pair_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                            const typename ExtraDstParam<GATHER>::type& extra, const GemmParams& p, int clusters,
                            cudaStream_t stream) {
    auto kernel = gemm_tcgen05_pair_kernel<KIND, OUT, GATHER, BN, ONE>;
    constexpr int smem = PairSmemT<BN, ONE>::kDynamicBytes;
    static_assert(smem <= 227 * 1024, "dynamic shared memory of one CTA");
    static bool configured[64] = {};
    static int max_clusters[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 74;
        }
        max_clusters[dev] = n;
        configured[dev] = true;
    }
    if (clusters > max_clusters[dev]) clusters = max_clusters[dev];
    if (clusters < 1) clusters = 1;
    if constexpr (ONE) {  // fewer clusters than tiles after all: the layout that allows several tiles per cluster
        if (clusters < p.total_work)
            return launch_pair_one<KIND, OUT, GATHER, BN, false>(ta, tb, tc, tws, extra, p, clusters, stream);
    }
    return launch_pdl(kernel, dim3(2 * clusters), dim3(kGemmThreads), smem, stream, ta, tb, tc, tws, extra, p);
}

// `bn` = 256, or 128 for the 256 x 128 tiles (one destination only).
template <int KIND>
cudaError_t launch_pair_kind(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                             const CUtensorMap& tws, const ExtraDst* extra, const GemmParams& p, int clusters,
                             cudaStream_t stream, bool one_ok = true) {
    const NoExtraDst none = {0};
    if (bn == 128 && one_ok && p.total_work <= clusters) {  // one tile per cluster: the nine-stage layout
        if (extra != nullptr) return cudaErrorInvalidValue;
        switch (out) {
            case OUT_F32: return launch_pair_one<KIND, OUT_F32, false, 128, true>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_BF16: return launch_pair_one<KIND, OUT_BF16, false, 128, true>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_F16: return launch_pair_one<KIND, OUT_F16, false, 128, true>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_RAW32: return launch_pair_one<KIND, OUT_RAW32, false, 128, true>(ta, tb, tc, tws, none, p, clusters, stream);
            default: return cudaErrorInvalidValue;
        }
    }
    if (bn == 128) {
        if (extra != nullptr) return cudaErrorInvalidValue;
        switch (out) {
            case OUT_F32: return launch_pair_one<KIND, OUT_F32, false, 128>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_BF16: return launch_pair_one<KIND, OUT_BF16, false, 128>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_F16: return launch_pair_one<KIND, OUT_F16, false, 128>(ta, tb, tc, tws, none, p, clusters, stream);
            case OUT_RAW32: return launch_pair_one<KIND, OUT_RAW32, false, 128>(ta, tb, tc, tws, none, p, clusters, stream);
            default: return cudaErrorInvalidValue;
        }
    }
#define QGEMM_PAIR_CASE(OUT_)                                                                            \
    case OUT_:                                                                                           \
        return extra ? launch_pair_one<KIND, OUT_, true>(ta, tb, tc, tws, *extra, p, clusters, stream)        \
                     : launch_pair_one<KIND, OUT_, false>(ta, tb, tc, tws, none, p, clusters, stream);
    switch (out) {
        QGEMM_PAIR_CASE(OUT_F32)
        QGEMM_PAIR_CASE(OUT_BF16)
        QGEMM_PAIR_CASE(OUT_F16)
        QGEMM_PAIR_CASE(OUT_RAW32)
        default: return cudaErrorInvalidValue;
    }
#undef QGEMM_PAIR_CASE
}

// Wide CTA-pair kernel (512 x 256 tiles per cluster of two; gemm_sm100_2cta_wide.cuh).
template <int KIND, int OUT>
cudaError_t launch_wide_one(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int clusters, cudaStream_t stream) {
    auto kernel = gemm_tcgen05_wide_pair_kernel<KIND, OUT>;
    constexpr int smem = WideSmem::kDynamicBytes;
    static bool configured[64] = {};
    static int max_clusters[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!configured[dev]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 74);
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = 74;
        }
        max_clusters[dev] = n;
        configured[dev] = true;
    }
    if (clusters > max_clusters[dev]) clusters = max_clusters[dev];
    if (clusters < 1) clusters = 1;
    return launch_pdl(kernel, dim3(2 * clusters), dim3(kGemmThreads), smem, stream, ta, tb, tc, p);
}

template <int KIND>
cudaError_t launch_wide_kind(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                             const GemmParams& p, int clusters, cudaStream_t stream) {
    switch (out) {
        case OUT_F32: return launch_wide_one<KIND, OUT_F32>(ta, tb, tc, p, clusters, stream);
        case OUT_BF16: return launch_wide_one<KIND, OUT_BF16>(ta, tb, tc, p, clusters, stream);
        case OUT_F16: return launch_wide_one<KIND, OUT_F16>(ta, tb, tc, p, clusters, stream);
        case OUT_RAW32: return launch_wide_one<KIND, OUT_RAW32>(ta, tb, tc, p, clusters, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemm_wide_f16(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                                 int clusters, cudaStream_t stream);
cudaError_t launch_gemm_wide_i8(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                                int clusters, cudaStream_t stream);
cudaError_t launch_gemm_wide_f8(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                                int clusters, cudaStream_t stream);

cudaError_t launch_gemm_pair_f16(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                                 const ExtraDst* extra, const GemmParams& p,
                                 int clusters, cudaStream_t stream, bool one_ok = true);
cudaError_t launch_gemm_pair_i8(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                                 const ExtraDst* extra, const GemmParams& p,
                                int clusters, cudaStream_t stream, bool one_ok = true);
cudaError_t launch_gemm_pair_f8(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                                 const ExtraDst* extra, const GemmParams& p,
                                int clusters, cudaStream_t stream, bool one_ok = true);

// Block-scaled FP8 GEMM (gemm_blockscale.cu): 128 x 128 tiles, one partial accumulator per 128-wide K block.
struct BlockScaleParams {
    void* C;
    long long ldc;
    int M, N, K;
    int m_tiles, n_tiles;
    int group_m;         // tile rows per scheduling group
    int kb_total;        // 128-element K blocks
    int n_scale_blocks;  // ceil(N / 128): row length of b_scale
    uint32_t idesc;
    const float* a_scale;  // [kb_total][M]
    const float* b_scale;  // [kb_total][n_scale_blocks]
    int* status;
    int c_tma_ok;
};
cudaError_t launch_fp8_blockscale(int out_kind, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                                  const BlockScaleParams& p, int grid, cudaStream_t stream);

// Adds up the K slices of the last-wave tiles (splitk_reduce.cu): `slots` tiles stored as
// [splits][slots * 256][tile_n] 32-bit partial sums (tile_n = 256 or 128, the pair kernel's tile width); `tiles`
// locates slot i in C (m_tiles, n_tiles, group_m, tile_offset; splits = 1).
int splitk_reduce_tiles_launch(const void* partials, int slots, int splits, bool acc_is_int, void* C, long long ldc,
                               int M, int N, int out_kind, const float* scale_a, const float* scale_b,
                               const GemmParams& tiles, int tile_n, cudaStream_t stream);

// Adds up the pieces of runs (GemmParams::sk_parts; splitk_reduce.cu): 2 * sk_parts slots of 256 x 256 partial sums;
// `tiles` carries sk_parts, sk_tiles, kb_total and the tile order (m_tiles, n_tiles, group_m; splits = 1).
int splitk_reduce_runs_launch(const void* partials, bool acc_is_int, void* C, long long ldc, int M, int N, int out_kind,
                              const float* scale_a, const float* scale_b, const GemmParams& tiles, cudaStream_t stream);

// In-cluster split-K (gemm_sm100_kcluster.cuh; gemm_kc_*.cu): `tiles` clusters of `slices` CTAs, 64- or 128-wide tiles.
cudaError_t launch_gemm_kcluster_f16(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                     const GemmParams& p, int tiles, cudaStream_t stream);
cudaError_t launch_gemm_kcluster_i8(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                    const GemmParams& p, int tiles, cudaStream_t stream);
cudaError_t launch_gemm_kcluster_f8(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                    const GemmParams& p, int tiles, cudaStream_t stream);
// The same for CTA pairs on 256 x 128 tiles (gemm_sm100_2cta_kcluster.cuh): `tiles` clusters of 2 * `slices` CTAs.
cudaError_t launch_gemm_pair_kcluster_f16(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                          const GemmParams& p, int tiles, cudaStream_t stream);
cudaError_t launch_gemm_pair_kcluster_i8(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                         const GemmParams& p, int tiles, cudaStream_t stream);
cudaError_t launch_gemm_pair_kcluster_f8(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                         const GemmParams& p, int tiles, cudaStream_t stream);
// Clusters of `slices` CTAs the current device keeps resident at once; 0 = unknown (no device).
int kcluster_max_clusters(int slices);

// Defined one per translation unit so the kinds compile in parallel.
cudaError_t launch_gemm_f16(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int grid, cudaStream_t stream, bool one = false);
cudaError_t launch_gemm_i8(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int grid, cudaStream_t stream, bool one = false);
cudaError_t launch_gemm_f8(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int grid, cudaStream_t stream, bool one = false);

}  // namespace qgemm
