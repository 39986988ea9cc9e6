// Matrix transpose / relayout for 1- and 2-byte elements: out[c*ld_out + r] = in[r*ld_in + c].
//
// Capability of the reference's src/transpose/transpose.cu:11-77 (bf16 only, 64x32 tiles, no bounds
// checks, element-wise bank-conflicted shared-memory writes), rebuilt for an HBM-bound kernel:
//   * every thread loads a B x B block of elements as B 16-byte vectors (B = 16 / sizeof(T): 8 x 8
//     for 2-byte, 16 x 16 for 1-byte elements), with the lanes of a warp side by side along the row
//     so each load instruction covers 256 contiguous bytes;
//   * the block is transposed in registers with byte permutes (no shared-memory element traffic);
//   * the B transposed vectors go through a shared-memory tile, XOR-swizzled in 16-byte units so that
//     both the writes (lanes spread over output rows) and the reads (lanes side by side along an
//     output row) are bank-conflict free;
//   * every thread then stores 16-byte vectors with the lanes side by side along the output row.
// Ragged edges and unaligned bases / leading dimensions take a guarded element-wise path per block.
//
// Algorithmic traffic: 2 * rows * cols * sizeof(T) bytes.
#include <cuda_runtime.h>
#include <cstdint>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

// Geometry per element size ES: B = elements per 16 bytes; a CTA of TBR x TBC threads covers
// (TBR*B) rows x (TBC*B) columns of the input.
template <int ES>
struct TransposeGeom {
    static constexpr int B = 16 / ES;
    static constexpr int TBC = 16;                  // thread columns: 16 lanes x 16 B = 256 B per row segment
    static constexpr int TBR = (ES == 2) ? 16 : 8;  // thread rows
    static constexpr int THREADS = TBR * TBC;
    static constexpr int TILE_R = TBR * B;          // 128 rows
    static constexpr int TILE_C = TBC * B;          // 128 (2-byte) or 256 (1-byte) columns
    static constexpr int UNITS_PER_OUT_ROW = TBR;   // 16-byte units along one output row of the tile
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// in[r] = row r of the block (B elements = 4 words); out[c] = column c of the block.
__device__ __forceinline__ void transpose_block_2byte(const uint4 (&in)[8], uint4 (&out)[8]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(in);  // w[r*4 + j]: elements 2j, 2j+1 of row r
    uint32_t* o = reinterpret_cast<uint32_t*>(out);             // o[c*4 + j]: rows 2j, 2j+1 of column c
#pragma unroll
    for (int c = 0; c < 8; ++c) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = w[(2 * j) * 4 + c / 2];
            const uint32_t hi = w[(2 * j + 1) * 4 + c / 2];
            o[c * 4 + j] = prmt(lo, hi, (c & 1) ? 0x7632u : 0x5410u);
        }
    }
}

__device__ __forceinline__ void transpose_block_1byte(const uint4 (&in)[16], uint4 (&out)[16]) {
    const uint32_t* w = reinterpret_cast<const uint32_t*>(in);  // w[r*4 + j]: bytes 4j..4j+3 of row r
    uint32_t* o = reinterpret_cast<uint32_t*>(out);             // o[c*4 + j]: rows 4j..4j+3 of column c
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        const int wi = c / 4, bi = c % 4;
        const uint32_t sel2 = static_cast<uint32_t>(bi) | (static_cast<uint32_t>(4 + bi) << 4);  // 2 bytes
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t t01 = prmt(w[(4 * j) * 4 + wi], w[(4 * j + 1) * 4 + wi], sel2);
            const uint32_t t23 = prmt(w[(4 * j + 2) * 4 + wi], w[(4 * j + 3) * 4 + wi], sel2);
            o[c * 4 + j] = prmt(t01, t23, 0x5410u);
        }
    }
}

template <int ES>
__global__ void __launch_bounds__(TransposeGeom<ES>::THREADS)
transpose_kernel(const void* __restrict__ in_v, void* __restrict__ out_v, int rows, int cols, long long ld_in,
                 long long ld_out, int in_vec_ok, int out_vec_ok) {
    using G = TransposeGeom<ES>;
    constexpr int B = G::B;
    constexpr int UR = G::UNITS_PER_OUT_ROW;
    __shared__ uint4 tile[G::TILE_C * UR];  // out-row c, unit u lives at c*UR + (u ^ ((c / B) % UR))

    const uint8_t* __restrict__ in = reinterpret_cast<const uint8_t*>(in_v);
    uint8_t* __restrict__ out = reinterpret_cast<uint8_t*>(out_v);
    const long long r0 = static_cast<long long>(blockIdx.y) * G::TILE_R;
    const long long c0 = static_cast<long long>(blockIdx.x) * G::TILE_C;
    const int tid = threadIdx.x;
    const int bc = tid % G::TBC;  // block column of this thread (lanes side by side along the row)
    const int br = tid / G::TBC;  // block row

    ptx::pdl_launch_dependents();
    ptx::pdl_wait();

    // ---- load the B x B block: rows r0 + br*B + i, columns c0 + bc*B .. +B-1
    uint4 blk[B];
    const long long gc = c0 + static_cast<long long>(bc) * B;
    const long long gr = r0 + static_cast<long long>(br) * B;
    if (in_vec_ok && gc + B <= cols && gr + B <= rows) {
#pragma unroll
        for (int i = 0; i < B; ++i)
            blk[i] = __ldg(reinterpret_cast<const uint4*>(in + ((gr + i) * ld_in + gc) * ES));
    } else {
#pragma unroll
        for (int i = 0; i < B; ++i) {
            alignas(16) uint8_t tmp[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const long long col = gc + e / ES;
                tmp[e] = (gr + i < rows && col < cols) ? in[((gr + i) * ld_in + col) * ES + e % ES] : uint8_t(0);
            }
            blk[i] = *reinterpret_cast<uint4*>(tmp);
        }
    }

    // ---- transpose in registers, park the B column-vectors in shared memory
    uint4 tr[B];
    if constexpr (ES == 2) transpose_block_2byte(blk, tr);
    else transpose_block_1byte(blk, tr);
#pragma unroll
    for (int i = 0; i < B; ++i) {
        const int c = bc * B + i;  // output row inside the tile; (c / B) % UR == bc % UR
        tile[c * UR + (br ^ (bc % UR))] = tr[i];
    }
    __syncthreads();

    // ---- store: unit index k -> output row c = k / UR, unit u = k % UR (lanes side by side along the row)
    constexpr int UNITS = G::TILE_C * UR;
#pragma unroll
    for (int k0 = 0; k0 < UNITS; k0 += G::THREADS) {
        const int k = k0 + tid;
        const int c = k / UR, u = k % UR;
        const uint4 v = tile[c * UR + (u ^ ((c / B) % UR))];
        const long long oc = c0 + c;                              // output row = input column
        const long long orow = r0 + static_cast<long long>(u) * B;  // first of the B input rows in this unit
        if (oc < cols && orow < rows) {
            if (out_vec_ok && orow + B <= rows) {
                *reinterpret_cast<uint4*>(out + (oc * ld_out + orow) * ES) = v;
            } else {
                alignas(16) uint8_t tmp[16];
                *reinterpret_cast<uint4*>(tmp) = v;
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (orow + e / ES < rows) out[(oc * ld_out + orow) * ES + e] = tmp[e];
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
    const int tile_r = 128;
    const int tile_c = (elem_bytes == 2) ? TransposeGeom<2>::TILE_C : TransposeGeom<1>::TILE_C;
    const size_t gx = (cols + tile_c - 1) / tile_c, gy = (rows + tile_r - 1) / tile_r;
    if (gy > 65535) return QGEMM_ERR_UNSUPPORTED;
    const int in_vec_ok = (reinterpret_cast<uintptr_t>(in) % 16 == 0) && ((ld_in * elem_bytes) % 16 == 0);
    const int out_vec_ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ld_out * elem_bytes) % 16 == 0);
    dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
    cudaError_t e;
    if (elem_bytes == 2)
        e = launch_pdl(transpose_kernel<2>, grid, dim3(TransposeGeom<2>::THREADS), 0, stream, in, out, (int)rows,
                       (int)cols, (long long)ld_in, (long long)ld_out, in_vec_ok, out_vec_ok);
    else
        e = launch_pdl(transpose_kernel<1>, grid, dim3(TransposeGeom<1>::THREADS), 0, stream, in, out, (int)rows,
                       (int)cols, (long long)ld_in, (long long)ld_out, in_vec_ok, out_vec_ok);
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace qgemm
