// In-cluster split-K kernel (gemm_sm100_kcluster.cuh), tcgen05 kind of the i8 operands.
#include "gemm_kcluster_launch.cuh"

namespace qgemm {
cudaError_t launch_gemm_kcluster_i8(int bn, int out, int am, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                    const GemmParams& p, int tiles, cudaStream_t stream) {
    return launch_kcluster_kind<ptx::KIND_I8>(bn, out, am, slices, ta, tb, p, tiles, stream);
}
cudaError_t launch_gemm_pair_kcluster_i8(int out, int slices, const CUtensorMap& ta, const CUtensorMap& tb,
                                         const GemmParams& p, int tiles, cudaStream_t stream) {
    return launch_pair_kcluster_kind<ptx::KIND_I8>(out, slices, ta, tb, p, tiles, stream);
}
}  // namespace qgemm
