// tcgen05 kind::f16 instantiations of the persistent GEMM kernel.
#include "gemm_launch.cuh"

namespace qgemm {
cudaError_t launch_gemm_f16(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int grid, cudaStream_t stream, bool one) {
    return launch_kind<ptx::KIND_F16>(bn, out, am, ta, tb, tc, p, grid, stream, one);
}
cudaError_t launch_gemm_pair_f16(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                                 const ExtraDst* extra,
                                 const GemmParams& p, int clusters, cudaStream_t stream, bool one_ok) {
    return launch_pair_kind<ptx::KIND_F16>(bn, out, ta, tb, tc, tws, extra, p, clusters, stream, one_ok);
}
cudaError_t launch_gemm_wide_f16(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                                 int clusters, cudaStream_t stream) {
    return launch_wide_kind<ptx::KIND_F16>(out, ta, tb, tc, p, clusters, stream);
}
}  // namespace qgemm
