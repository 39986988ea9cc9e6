// In-cluster split-K kernel (gemm_sm100_kcluster.cuh), tcgen05 kind of the f8 operands.
#include "gemm_kcluster_launch.cuh"

namespace qgemm {
cudaError_t launch_gemm_kcluster_f8(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                    const GemmParams& p, int tiles, cudaStream_t stream) {
    return launch_kcluster_kind<ptx::KIND_F8>(bn, out, am, slices, ta, tb, p, tiles, stream);
}
cudaError_t launch_gemm_pair_kcluster_f8(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                         const GemmParams& p, int tiles, cudaStream_t stream) {
    return launch_pair_kcluster_kind<ptx::KIND_F8>(out, slices, ta, tb, p, tiles, stream);
}

// How many clusters of `slices` CTAs of this kernel the current device keeps resident at once (a cluster needs its
// CTAs on SMs of one GPC, so this is less than SMs / slices); 0 when it cannot be asked (no device). Asked once per
// device and cluster size, on the instantiation with the largest shared-memory footprint.
template <int S>
static int max_clusters_of() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        (void)cudaGetLastError();
        return 0;
    }
    if (cached[dev] != 0) return cached[dev];
    constexpr int STAGES = StagesFor<128, 128>::value + 1;
    auto kernel = gemm_tcgen05_kcluster_kernel<ptx::KIND_F8, 128, STAGES, OUT_BF16, 128, S>;
    constexpr int smem = GemmSmem<128, STAGES, 128, true>::kDynamicBytes;
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(S * 32);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return 0;
    }
    cached[dev] = n;
    return n;
}
int kcluster_max_clusters(int slices) {
    switch (slices) {
        case 2: return max_clusters_of<2>();
        case 4: return max_clusters_of<4>();
        case 8: return max_clusters_of<8>();
        default: return 0;
    }
}
}  // namespace qgemm
