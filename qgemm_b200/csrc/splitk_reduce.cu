// Second pass of split-K: a deterministic, fixed-order sum of the per-split partial accumulators
// followed by the same scale + down-cast the fused epilogue applies. The reference only sketches
// split-K (an unused `split_k` constant, src/gemm/sm89_gemm_kernel_v5.cu:319); int8 partials are
// kept as int32 so the split path stays bit-exact.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

// Sums four consecutive columns over the splits (src, src + split_stride, ...) in split order and writes
// cast(scale_a * scale_b * sum), or the raw 32-bit sum, to C[row, col .. col+3] (columns >= N left alone).
template <bool ACC_INT>
__device__ __forceinline__ void reduce_quad(const uint32_t* __restrict__ src, long long split_stride, int splits,
                                            void* __restrict__ C, long long ldc, long long row, int col, int N,
                                            int out_kind, const float* __restrict__ scale_a,
                                            const float* __restrict__ scale_b, int c_vec_ok,
                                            const uint32_t* __restrict__ first_src = nullptr) {
    // first_src != nullptr: term 0 is read there instead of at src (the other terms stay at src + k * split_stride)
    uint32_t raw[4];
    float f[4];
    if constexpr (ACC_INT) {
        int s[4] = {0, 0, 0, 0};
        for (int k = 0; k < splits; ++k) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>((k == 0 && first_src != nullptr) ? first_src : src + k * split_stride));
            s[0] += static_cast<int>(v.x);
            s[1] += static_cast<int>(v.y);
            s[2] += static_cast<int>(v.z);
            s[3] += static_cast<int>(v.w);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            raw[j] = static_cast<uint32_t>(s[j]);
            f[j] = static_cast<float>(s[j]);
        }
    } else {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < splits; ++k) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>((k == 0 && first_src != nullptr) ? first_src : src + k * split_stride));
            s[0] += __uint_as_float(v.x);
            s[1] += __uint_as_float(v.y);
            s[2] += __uint_as_float(v.z);
            s[3] += __uint_as_float(v.w);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            raw[j] = __float_as_uint(s[j]);
            f[j] = s[j];
        }
    }

    const int n_valid = min(4, N - col);
    if (out_kind == OUT_RAW32) {
        uint32_t* dst = reinterpret_cast<uint32_t*>(C) + row * ldc + col;
        if (c_vec_ok && n_valid == 4) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
        } else {
            for (int j = 0; j < n_valid; ++j) dst[j] = raw[j];
        }
        return;
    }
    float alpha = 1.0f;
    if (scale_a != nullptr) alpha *= __ldg(scale_a);
    if (scale_b != nullptr) alpha *= __ldg(scale_b);
#pragma unroll
    for (int j = 0; j < 4; ++j) f[j] *= alpha;
    if (out_kind == OUT_F32) {
        float* dst = reinterpret_cast<float*>(C) + row * ldc + col;
        if (c_vec_ok && n_valid == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
        } else {
            for (int j = 0; j < n_valid; ++j) dst[j] = f[j];
        }
    } else {
        uint16_t h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (out_kind == OUT_BF16) {
                __nv_bfloat16 b = __float2bfloat16_rn(f[j]);
                h[j] = *reinterpret_cast<uint16_t*>(&b);
            } else {
                __half b = __float2half_rn(f[j]);
                h[j] = *reinterpret_cast<uint16_t*>(&b);
            }
        }
        uint16_t* dst = reinterpret_cast<uint16_t*>(C) + row * ldc + col;
        if (c_vec_ok && n_valid == 4) {
            *reinterpret_cast<uint2*>(dst) =
                make_uint2(h[0] | (static_cast<uint32_t>(h[1]) << 16), h[2] | (static_cast<uint32_t>(h[3]) << 16));
        } else {
            for (int j = 0; j < n_valid; ++j) dst[j] = h[j];
        }
    }
}

template <bool ACC_INT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const uint32_t* __restrict__ partials, long long split_stride, long long ldw, int splits,
                     void* __restrict__ C, long long ldc, int M, int N, int out_kind,
                     const float* __restrict__ scale_a, const float* __restrict__ scale_b, int c_vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    // blockIdx.x walks along a row (four columns per thread), blockIdx.y strides over the rows: no per-thread division
    const int col = (static_cast<int>(blockIdx.x) * static_cast<int>(blockDim.x) + static_cast<int>(threadIdx.x)) * 4;
    if (col >= N) return;
    for (long long row = blockIdx.y; row < M; row += gridDim.y)
        reduce_quad<ACC_INT>(partials + row * ldw + col, split_stride, splits, C, ldc, row, col, N, out_kind, scale_a,
                             scale_b, c_vec_ok);
}

// The same sum for tiles whose K slices were stored as compact 256 x tile_n slots ([splits][slots * 256][tile_n],
// tile_n = 256 or 128): blockIdx.y = slot; the tile's place in C comes from the GEMM's own tile order (`tiles`
// carries m_tiles, n_tiles, group_m and tile_offset, with splits = 1).
template <bool ACC_INT>
__global__ void __launch_bounds__(256)
splitk_reduce_tiles_kernel(const uint32_t* __restrict__ partials, long long split_stride, int splits,
                           void* __restrict__ C, long long ldc, int M, int N, int out_kind,
                           const float* __restrict__ scale_a, const float* __restrict__ scale_b, int c_vec_ok,
                           const GemmParams tiles, int tile_n) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const int slot = static_cast<int>(blockIdx.y);
    const TileCoord t = decode_tile(slot, tiles);
    const int idx = static_cast<int>(blockIdx.x) * 256 + static_cast<int>(threadIdx.x);  // 256 rows x tile_n / 4 quads
    const int quad_shift = tile_n == 256 ? 6 : 5;
    const int r = idx >> quad_shift;
    const int c = (idx & ((1 << quad_shift) - 1)) * 4;
    const long long row = static_cast<long long>(t.m_blk) * kPairTileM + r;
    const int col = t.n_blk * tile_n + c;
    if (r >= kPairTileM || row >= M || col >= N) return;
    const uint32_t* src = partials + (static_cast<long long>(slot) * kPairTileM + r) * tile_n + c;
    reduce_quad<ACC_INT>(src, split_stride, splits, C, ldc, row, col, N, out_kind, scale_a, scale_b, c_vec_ok);
}

// The same sum for the pieces of runs (GemmParams::sk_parts): blockIdx.y = tile; the tile's K blocks [t * kb, (t + 1) * kb)
// of the end-to-end order lie in runs first ... last, one piece each, in run order. A piece that begins its run lies in
// scratch slot [run], one that does not (it began at the tile's first block) in slot [parts + run]; slots are 256 x 256
// partial sums. A tile that lies in one run was stored to C by the GEMM itself.
template <bool ACC_INT>
__global__ void __launch_bounds__(256)
splitk_reduce_runs_kernel(const uint32_t* __restrict__ partials, void* __restrict__ C, long long ldc, int M, int N,
                          int out_kind, const float* __restrict__ scale_a, const float* __restrict__ scale_b,
                          int c_vec_ok, const GemmParams tiles) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const int tile = static_cast<int>(blockIdx.y);
    const long long total = static_cast<long long>(tiles.sk_tiles) * tiles.kb_total;
    const long long begin = static_cast<long long>(tile) * tiles.kb_total;
    const int first = run_of_block(begin, tiles.sk_parts, total);
    const int last = run_of_block(begin + tiles.kb_total - 1, tiles.sk_parts, total);
    if (first == last) return;
    const TileCoord t = decode_tile(tile, tiles);
    const int idx = static_cast<int>(blockIdx.x) * 256 + static_cast<int>(threadIdx.x);  // 256 rows x 64 quads
    const int r = idx >> 6;
    const int c = (idx & 63) * 4;
    const long long row = static_cast<long long>(t.m_blk) * kPairTileM + r;
    const int col = t.n_blk * kPairTileN + c;
    if (r >= kPairTileM || row >= M || col >= N) return;
    const long long slot_elems = static_cast<long long>(kPairTileM) * kPairTileN;
    const long long in_slot = static_cast<long long>(r) * kPairTileN + c;
    const bool first_begins_here = (first * total) / tiles.sk_parts == begin;
    const uint32_t* first_src = partials + (first_begins_here ? first : tiles.sk_parts + first) * slot_elems + in_slot;
    const uint32_t* src = partials + first * slot_elems + in_slot;  // src + k * slot_elems: the piece that begins run first + k
    reduce_quad<ACC_INT>(src, slot_elems, last - first + 1, C, ldc, row, col, N, out_kind, scale_a, scale_b, c_vec_ok,
                         first_src);
}

}  // namespace

int splitk_reduce_runs_launch(const void* partials, bool acc_is_int, void* C, long long ldc, int M, int N, int out_kind,
                              const float* scale_a, const float* scale_b, const GemmParams& tiles, cudaStream_t stream) {
    if (tiles.sk_tiles <= 0 || tiles.sk_parts <= 0) return QGEMM_OK;
    const int out_bytes = (out_kind == OUT_BF16 || out_kind == OUT_F16) ? 2 : 4;
    const int c_vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && ((ldc * out_bytes) % 16 == 0);
    const uint32_t* p = reinterpret_cast<const uint32_t*>(partials);
    const dim3 grid(kPairTileM * (kPairTileN / 4) / 256, static_cast<unsigned>(tiles.sk_tiles));
    cudaError_t e;
    if (acc_is_int)
        e = launch_pdl(splitk_reduce_runs_kernel<true>, grid, dim3(256), 0, stream, p, C, ldc, M, N, out_kind, scale_a,
                       scale_b, c_vec_ok, tiles);
    else
        e = launch_pdl(splitk_reduce_runs_kernel<false>, grid, dim3(256), 0, stream, p, C, ldc, M, N, out_kind, scale_a,
                       scale_b, c_vec_ok, tiles);
    return e == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

int splitk_reduce_tiles_launch(const void* partials, int slots, int splits, bool acc_is_int, void* C, long long ldc,
                               int M, int N, int out_kind, const float* scale_a, const float* scale_b,
                               const GemmParams& tiles, int tile_n, cudaStream_t stream) {
    if (slots <= 0) return QGEMM_OK;
    if (tile_n != 256 && tile_n != 128) return QGEMM_ERR_INVALID_ARG;
    const int out_bytes = (out_kind == OUT_BF16 || out_kind == OUT_F16) ? 2 : 4;
    const int c_vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && ((ldc * out_bytes) % 16 == 0);
    const long long split_stride = static_cast<long long>(slots) * kPairTileM * tile_n;
    const uint32_t* p = reinterpret_cast<const uint32_t*>(partials);
    const dim3 grid(kPairTileM * (tile_n / 4) / 256, static_cast<unsigned>(slots));
    cudaError_t e;
    if (acc_is_int)
        e = launch_pdl(splitk_reduce_tiles_kernel<true>, grid, dim3(256), 0, stream, p, split_stride, splits, C, ldc, M,
                       N, out_kind, scale_a, scale_b, c_vec_ok, tiles, tile_n);
    else
        e = launch_pdl(splitk_reduce_tiles_kernel<false>, grid, dim3(256), 0, stream, p, split_stride, splits, C, ldc,
                       M, N, out_kind, scale_a, scale_b, c_vec_ok, tiles, tile_n);
    return e == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

int splitk_reduce_launch(const void* partials, long long split_stride, long long ldw, int splits, bool acc_is_int,
                         void* C, long long ldc, int M, int N, int out_kind, const float* scale_a,
                         const float* scale_b, cudaStream_t stream) {
    const int out_bytes = (out_kind == OUT_BF16 || out_kind == OUT_F16) ? 2 : 4;
    const int c_vec_ok = (reinterpret_cast<uintptr_t>(C) % 16 == 0) && ((ldc * out_bytes) % 16 == 0);
    if (M <= 0 || N <= 0) return QGEMM_OK;
    const int threads = 256;
    const unsigned blocks_x = static_cast<unsigned>(((N + 3) / 4 + threads - 1) / threads);
    const unsigned blocks_y = static_cast<unsigned>(std::min<long long>(M, 65535));
    const dim3 grid(blocks_x, blocks_y);
    const uint32_t* p = reinterpret_cast<const uint32_t*>(partials);
    cudaError_t e;
    if (acc_is_int)
        e = launch_pdl(splitk_reduce_kernel<true>, grid, dim3(threads), 0, stream, p, split_stride, ldw, splits, C, ldc, M,
                       N, out_kind, scale_a, scale_b, c_vec_ok);
    else
        e = launch_pdl(splitk_reduce_kernel<false>, grid, dim3(threads), 0, stream, p, split_stride, ldw, splits, C, ldc, M,
                       N, out_kind, scale_a, scale_b, c_vec_ok);
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;
    return cudaGetLastError() == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace qgemm
