// tcgen05 kind::f8f6f4 instantiations of the persistent GEMM kernel.
#include "gemm_launch.cuh"

namespace qgemm {
cudaError_t launch_gemm_f8(int bn, int out, int am, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                            int grid, cudaStream_t stream, bool one) {
    return launch_kind<ptx::KIND_F8>(bn, out, am, ta, tb, tc, p, grid, stream, one);
}
cudaError_t launch_gemm_pair_f8(int bn, int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tws,
                                 const ExtraDst* extra,
                                 const GemmParams& p, int clusters, cudaStream_t stream, bool one_ok) {
    return launch_pair_kind<ptx::KIND_F8>(bn, out, ta, tb, tc, tws, extra, p, clusters, stream, one_ok);
}
cudaError_t launch_gemm_wide_f8(int out, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                                 int clusters, cudaStream_t stream) {
    return launch_wide_kind<ptx::KIND_F8>(out, ta, tb, tc, p, clusters, stream);
}
}  // namespace qgemm

#ifdef QGEMM_STAMPS
// Diagnostic build only: the cycle stamps of the last FP8 lone-CTA launch ([first CTA | last CTA] x 16).
extern "C" int qgemm_debug_stamps(long long* out32) {
    return cudaMemcpyFromSymbol(out32, qgemm::g_stamps, sizeof(long long) * 32) == cudaSuccess ? 0 : 4;
}
#endif
