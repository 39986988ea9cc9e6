// Matrix transpose / relayout for 1- and 2-byte elements: out[c*ld_out + r] = in[r*ld_in + c].
//
// Capability of the reference's src/transpose/transpose.cu:11-77 (bf16 only, 64x32 tiles, no bounds
// checks, 2-byte bank-conflicted shared-memory writes), rebuilt: 128-bit global accesses on both
// sides, a shared-memory tile whose 16-byte units are XOR-swizzled so that both the row-wise vector
// writes and the column-wise element reads are bank-conflict free, any rows/cols/leading
// dimensions (ragged edges and unaligned bases take a guarded element-wise path per unit).
//
// It is HBM-bound: 2 * rows * cols * sizeof(T) bytes of algorithmic traffic.
#include <cuda_runtime.h>
#include <cstdint>

#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kTransposeThreads = 256;

// ES = element size in bytes. The tile is T x T elements with T * ES = 128 bytes per row, i.e.
// 8 sixteen-byte units per row; VEC = elements per unit.
template <int ES>
struct ElemT;
template <>
struct ElemT<1> {
    using type = uint8_t;
};
template <>
struct ElemT<2> {
    using type = uint16_t;
};

template <int ES>
__global__ void __launch_bounds__(kTransposeThreads)
transpose_kernel(const void* __restrict__ in_v, void* __restrict__ out_v, int rows, int cols, long long ld_in,
                 long long ld_out, int in_vec_ok, int out_vec_ok) {
    using E = typename ElemT<ES>::type;
    constexpr int T = 128 / ES;    // tile edge in elements
    constexpr int VEC = 16 / ES;   // elements per 16-byte unit
    constexpr int UNITS = T * 8;   // 16-byte units in the tile
    constexpr int PER_THREAD = UNITS / kTransposeThreads;
    __shared__ uint4 tile[UNITS];  // unit (r, u) lives at r*8 + (u ^ ((r / VEC) & 7))

    const E* __restrict__ in = reinterpret_cast<const E*>(in_v);
    E* __restrict__ out = reinterpret_cast<E*>(out_v);
    const long long r0 = static_cast<long long>(blockIdx.y) * T;
    const long long c0 = static_cast<long long>(blockIdx.x) * T;
    const int tid = threadIdx.x;

    // ---- global -> shared: unit index i -> row i/8, unit-in-row i%8 (8 lanes cover one 128-byte row)
    uint4 regs[PER_THREAD];
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = tid + j * kTransposeThreads;
        const int r = i >> 3, u = i & 7;
        const long long gr = r0 + r, gc = c0 + u * VEC;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (gr < rows) {
            if (in_vec_ok && gc + VEC <= cols) {
                val = __ldg(reinterpret_cast<const uint4*>(in + gr * ld_in + gc));
            } else {
                alignas(16) E tmp[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) tmp[e] = (gc + e < cols) ? in[gr * ld_in + gc + e] : E(0);
                val = *reinterpret_cast<uint4*>(tmp);
            }
        }
        regs[j] = val;
    }
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = tid + j * kTransposeThreads;
        const int r = i >> 3, u = i & 7;
        tile[r * 8 + (u ^ ((r / VEC) & 7))] = regs[j];
    }
    __syncthreads();

    // ---- shared -> global: output unit i -> output row (input column) c = i/8, unit-in-row ur = i%8
    //      holding input rows ur*VEC .. ur*VEC+VEC-1 of column c.
    const E* tile_e = reinterpret_cast<const E*>(tile);
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = tid + j * kTransposeThreads;
        const int c = i >> 3, ur = i & 7;
        const int cu = c / VEC, ce = c % VEC;
        alignas(16) E tmp[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const int r = ur * VEC + e;  // (r / VEC) & 7 == ur
            tmp[e] = tile_e[(r * 8 + (cu ^ ur)) * VEC + ce];
        }
        const long long gc = c0 + c, gr = r0 + ur * VEC;
        if (gc < cols && gr < rows) {
            if (out_vec_ok && gr + VEC <= rows) {
                *reinterpret_cast<uint4*>(out + gc * ld_out + gr) = *reinterpret_cast<uint4*>(tmp);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    if (gr + e < rows) out[gc * ld_out + gr + e] = tmp[e];
            }
        }
    }
}

}  // namespace

int transpose_launch(const void* in, void* out, size_t rows, size_t cols, size_t ld_in, size_t ld_out,
                     size_t elem_bytes, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return QGEMM_OK;
    if (in == nullptr || out == nullptr) return QGEMM_ERR_INVALID_ARG;
    if (ld_in < cols || ld_out < rows) return QGEMM_ERR_INVALID_ARG;
    if (elem_bytes != 1 && elem_bytes != 2) return QGEMM_ERR_UNSUPPORTED;
    if (rows > 0x7fffffffull || cols > 0x7fffffffull) return QGEMM_ERR_INVALID_ARG;
    const int tile = 128 / static_cast<int>(elem_bytes);
    const size_t gx = (cols + tile - 1) / tile, gy = (rows + tile - 1) / tile;
    if (gy > 65535) return QGEMM_ERR_UNSUPPORTED;
    const int in_vec_ok = (reinterpret_cast<uintptr_t>(in) % 16 == 0) && ((ld_in * elem_bytes) % 16 == 0);
    const int out_vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ld_out * elem_bytes) % 16 == 0);
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    if (elem_bytes == 2)
        transpose_kernel<2><<<grid, kTransposeThreads, 0, stream>>>(in, out, (int)rows, (int)cols, (long long)ld_in,
                                                                    (long long)ld_out, in_vec_ok, out_vec_ok);
    else
        transpose_kernel<1><<<grid, kTransposeThreads, 0, stream>>>(in, out, (int)rows, (int)cols, (long long)ld_in,
                                                                    (long long)ld_out, in_vec_ok, out_vec_ok);
    return cudaGetLastError() == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace qgemm
