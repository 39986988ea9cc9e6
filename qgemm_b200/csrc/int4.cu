// Signed 4-bit operands (the "Int4" precision of the reference's roadmap, develop.md:9-12; the reference has no
// int4 code). Storage: two values per byte, element 2i in the low nibble of byte i, two's complement (-8..7),
// rows K-major. The 5th-generation tensor cores have no 4-bit integer kind, so an int4 GEMM is the int8 GEMM
// (kind::i8, exact int32 accumulation) on operands widened by the pass below: HBM-bound, K/2 bytes in and K
// bytes out per row, 16-byte loads and stores.
#include <algorithm>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kUnpackThreads = 256;

// Eight nibbles of w -> eight sign-extended bytes, in element order, as two 32-bit words.
__device__ __forceinline__ void widen8(uint32_t w, uint32_t& lo4, uint32_t& hi4) {
    const uint32_t l = w & 0x0f0f0f0fu;          // elements 0, 2, 4, 6 (one per byte)
    const uint32_t h = (w >> 4) & 0x0f0f0f0fu;   // elements 1, 3, 5, 7
    // sign-extend 4 -> 8 bits per byte: (x ^ 8) - 8
    const uint32_t ls = __vsub4(l ^ 0x08080808u, 0x08080808u);
    const uint32_t hs = __vsub4(h ^ 0x08080808u, 0x08080808u);
    lo4 = __byte_perm(ls, hs, 0x5140);  // e0 e1 e2 e3
    hi4 = __byte_perm(ls, hs, 0x7362);  // e4 e5 e6 e7
}

// One thread widens 32 elements (16 packed bytes) of a row: blockIdx.x walks along the row, blockIdx.y strides over
// the rows (no per-thread division).
__global__ void __launch_bounds__(kUnpackThreads)
unpack_int4_kernel(const uint8_t* __restrict__ in, long long ld_in_bytes, int8_t* __restrict__ out, long long ld_out,
                   int rows, int cols, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const int c = (static_cast<int>(blockIdx.x) * kUnpackThreads + static_cast<int>(threadIdx.x)) * 32;
    if (c >= cols) return;
    for (long long r = blockIdx.y; r < rows; r += gridDim.y) {
        const uint8_t* src = in + r * ld_in_bytes + c / 2;
        int8_t* dst = out + r * ld_out + c;
        if (vec_ok && c + 32 <= cols) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
            uint4 a, b;
            widen8(v.x, a.x, a.y);
            widen8(v.y, a.z, a.w);
            widen8(v.z, b.x, b.y);
            widen8(v.w, b.z, b.w);
            reinterpret_cast<uint4*>(dst)[0] = a;
            reinterpret_cast<uint4*>(dst)[1] = b;
        } else {
            for (int e = 0; e < 32 && c + e < cols; ++e) {
                const uint8_t byte = src[e >> 1];
                const int nib = (e & 1) ? (byte >> 4) : (byte & 0x0f);
                dst[e] = static_cast<int8_t>((nib ^ 8) - 8);
            }
        }
    }
}

}  // namespace

int unpack_int4_launch(const void* in, size_t ld_in_elems, void* out, size_t ld_out, size_t rows, size_t cols,
                       cudaStream_t stream) {
    if (rows == 0 || cols == 0) return QGEMM_OK;
    if (in == nullptr || out == nullptr || (cols & 1) || (ld_in_elems & 1) || ld_in_elems < cols || ld_out < cols)
        return QGEMM_ERR_INVALID_ARG;
    if (rows > 0x7fffffffull || cols > 0x7fffffffull) return QGEMM_ERR_INVALID_ARG;
    const size_t ld_in_bytes = ld_in_elems / 2;
    const int vec_ok = (reinterpret_cast<uintptr_t>(in) % 16 == 0) && (ld_in_bytes % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (ld_out % 16 == 0);
    const unsigned blocks_x = static_cast<unsigned>(((cols + 31) / 32 + kUnpackThreads - 1) / kUnpackThreads);
    const unsigned blocks_y = static_cast<unsigned>(std::min<size_t>(rows, 65535));
    const cudaError_t e =
        launch_pdl(unpack_int4_kernel, dim3(blocks_x, blocks_y), dim3(kUnpackThreads), 0, stream,
                   static_cast<const uint8_t*>(in), static_cast<long long>(ld_in_bytes), static_cast<int8_t*>(out),
                   static_cast<long long>(ld_out), static_cast<int>(rows), static_cast<int>(cols), vec_ok);
    return e == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace qgemm
