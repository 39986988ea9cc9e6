// Per-matrix quantisation pre-pass: the step in front of the mixed GEMM. The reference's roadmap lists
// it (develop.md:9-12, README.md:1 "The input matrix will be quantized to 8 bits") but ships no kernel;
// the semantics are those of C = (A o Q_A) x (B o Q_B) (README.md:5-7) with one coefficient per matrix:
//   amax  = max |x|,  scale = amax / qmax  (qmax = 448 for FP8 e4m3, 127 for int8, 7 for packed int4; scale = 1
//           if amax == 0)
//   q     = round_to_nearest_even(x / scale), saturated to +-qmax,
// so that x ~= scale * q and `scale` is what the GEMM epilogue multiplies back in.
//
// Two HBM-bound passes over the input: an absolute-maximum reduction (warp shuffles, one atomicMax per
// block on the float's bit pattern, which orders like the value for non-negative floats) and the
// conversion pass, 16-byte loads where the layout allows.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kQuantThreads = 256;

template <typename TIn>
__device__ __forceinline__ float load_as_float(const TIn* p) {
    if constexpr (sizeof(TIn) == 4) return *reinterpret_cast<const float*>(p);
    else return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(p));
}

// Four consecutive elements of a row as floats (one 16-byte or 8-byte load).
template <typename TIn>
struct Quad {
    using Raw = typename std::conditional<sizeof(TIn) == 4, float4, uint2>::type;
    static __device__ __forceinline__ Raw load(const TIn* p) { return __ldg(reinterpret_cast<const Raw*>(p)); }
    static __device__ __forceinline__ void to_float(const Raw& v, float (&x)[4]) {
        if constexpr (sizeof(TIn) == 4) {
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
            x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
        }
    }
};

// Loads in flight per thread: both passes are plain streams, and with one small load per loop iteration the
// bytes in flight per SM (2048 threads x 8 or 16 bytes) are too few to cover HBM latency at full bandwidth.
template <typename TIn>
struct Unroll {
    static constexpr int value = sizeof(TIn) == 4 ? 4 : 8;
};

// Work decomposition of both passes: a block takes one *chunk* of a row at a time -- kQuantThreads x U quads of 4
// elements, thread t the quads t, t + kQuantThreads, ... of the chunk, so that every load instruction of a warp covers
// 512 (or 256) contiguous bytes and a thread has U loads in flight. Row and chunk come from one division per block and
// chunk, not one per element (a 64-bit division costs more than the rest of the per-element work together).
template <typename TIn>
__global__ void __launch_bounds__(kQuantThreads)
amax_kernel(const TIn* __restrict__ in, long long ld, int rows, int cols, float* __restrict__ amax_out, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    constexpr int U = Unroll<TIn>::value;
    constexpr int kChunkQuads = kQuantThreads * U;
    const int quads_per_row = (cols + 3) / 4;
    const int chunks_per_row = (quads_per_row + kChunkQuads - 1) / kChunkQuads;
    const long long items = static_cast<long long>(chunks_per_row) * rows;
    float m = 0.0f;
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
        const long long r = item / chunks_per_row;
        const int q0 = static_cast<int>(item - r * chunks_per_row) * kChunkQuads + static_cast<int>(threadIdx.x);
        const TIn* row = in + r * ld;
        if (vec_ok && (q0 + (U - 1) * kQuantThreads) * 4 + 4 <= cols) {
            typename Quad<TIn>::Raw v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = Quad<TIn>::load(row + (q0 + u * kQuantThreads) * 4);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float x[4];
                Quad<TIn>::to_float(v[u], x);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
            }
            continue;
        }
        for (int u = 0; u < U; ++u) {
            const int c = (q0 + u * kQuantThreads) * 4;
            if (c >= cols) break;
            if (vec_ok && c + 4 <= cols) {
                float x[4];
                Quad<TIn>::to_float(Quad<TIn>::load(row + c), x);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
            } else {
                for (int e = 0; e < 4 && c + e < cols; ++e) m = fmaxf(m, fabsf(load_as_float(row + c + e)));
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float warp_max[kQuantThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < kQuantThreads / 32 ? warp_max[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(m));
    }
}

// round_to_nearest_even(fl(x / scale)) as an integer, clamped to +-qmax -- the division's result without the division
// wherever that is provably the same. x * (1 / scale) is within 2^-23 relative, i.e. within 3e-5 for |q| <= 256, of
// the true quotient, and so is the correctly rounded quotient (1.5e-5); unless the product lies within 1e-4 of k + 1/2
// both round to the same integer. The rounding itself is the add-a-large-constant form (2^23 + 2^22: the sum's low
// mantissa bits are the integer, rounded to nearest even by the addition), so the common path has neither a division
// nor a float <-> int conversion, both of which issue at a fraction of the FP32 rate and bounded this pass below the
// HBM rate (bf16 -> int8: 3.97 TB/s of 6.5). The product is clamped just inside +-(qmax + 1/2) first, which saturates
// and keeps the constant trick in range; anything the clamp moved, ties, NaNs and scales whose reciprocal is not a
// normal number (the reciprocal is then set to NaN) fail the distance test and take the exact path.
struct QuotientRounder {
    float scale, rcp;
    __device__ __forceinline__ explicit QuotientRounder(float s) {
        scale = s;
        rcp = (s >= 1e-30f && s <= 1e30f) ? __fdiv_rn(1.0f, s) : __int_as_float(0x7fc00000);
    }
    // Returns a word whose LOW BYTE is the two's-complement result (the constant's own low byte is zero, so the sum's
    // bit pattern can be used as it is: no subtraction, no conversion).
    template <int QMAX>
    __device__ __forceinline__ uint32_t round_low_byte(float x) const {
        constexpr float kMagic = 12582912.0f;  // 2^23 + 2^22 = 0x4B400000
        constexpr float kLim = static_cast<float>(QMAX) + 0.49f;
        const float qf = x * rcp;
        const float t = fminf(fmaxf(qf, -kLim), kLim) + kMagic;
        const float n = t - kMagic;  // exact: the clamped product rounded to an integer in [-QMAX, QMAX]
        if (fabsf(qf - n) < 0.4999f) return __float_as_uint(t);
        return static_cast<uint32_t>(max(-QMAX, min(QMAX, __float2int_rn(__fdiv_rn(x, scale)))));
    }
    // Four int8 results packed into a word. Fused multiply-adds: t = RN(x * rcp + 2^23 + 2^22) carries the integer
    // nearest to the product, d = RN(x * rcp - n) its distance from it (one rounding each). No clamp: the scale is
    // amax / 127 of this very matrix (the library's own first pass), so |x * rcp| <= 127 (1 + 2^-22) and the integer
    // is within +-127 by construction; a NaN among the four fails the comparison and sends the quad down the exact path.
    __device__ __forceinline__ uint32_t round_quad_int8(const float (&x)[4]) const {
        constexpr float kMagic = 12582912.0f;
        float t[4];
        bool ok = true;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            t[j] = __fmaf_rn(x[j], rcp, kMagic);
            const float n = t[j] - kMagic;
            ok = ok && (fabsf(__fmaf_rn(x[j], rcp, -n)) < 0.4999f);
        }
        if (ok) {  // the four low bytes gathered with three byte permutes
            const uint32_t lo = __byte_perm(__float_as_uint(t[0]), __float_as_uint(t[1]), 0x0040);
            const uint32_t hi = __byte_perm(__float_as_uint(t[2]), __float_as_uint(t[3]), 0x0040);
            return __byte_perm(lo, hi, 0x5410);
        }
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            w |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(__fdiv_rn(x[j], scale))))) & 0xffu) << (8 * j);
        return w;
    }
};

template <bool FP8>
__device__ __forceinline__ uint8_t quantize_one(float x, const QuotientRounder& qr) {
    if constexpr (FP8) {
        return static_cast<uint8_t>(__nv_cvt_float_to_fp8(__fdiv_rn(x, qr.scale), __NV_SATFINITE, __NV_E4M3));
    } else {
        // round to nearest even straight to an integer (what rintf + cast does), then saturate to +-127
        return static_cast<uint8_t>(qr.round_low_byte<127>(x) & 0xffu);
    }
}

// Four quantised values packed into one 32-bit word.
template <bool FP8>
__device__ __forceinline__ uint32_t quantize_quad(const float (&x)[4], const QuotientRounder& qr) {
    const float scale = qr.scale;
    if constexpr (FP8) {
        // two values per conversion instruction (same rounding and saturation as the scalar form)
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x[0], scale), __fdiv_rn(x[1], scale)),
                                                     __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(x[2], scale), __fdiv_rn(x[3], scale)),
                                                     __NV_SATFINITE, __NV_E4M3);
        return lo | (hi << 16);
    } else {
        return qr.round_quad_int8(x);
    }
}

template <typename TIn, bool FP8>
__global__ void __launch_bounds__(kQuantThreads)
quantize_kernel(const TIn* __restrict__ in, long long ld_in, uint8_t* __restrict__ out, long long ld_out, int rows,
                int cols, const float* __restrict__ amax_in, float* __restrict__ scale_out, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    constexpr int U = Unroll<TIn>::value;
    constexpr int kChunkQuads = kQuantThreads * U;
    const float amax = __ldg(amax_in);
    const float qmax = FP8 ? 448.0f : 127.0f;
    const float scale = amax > 0.0f ? __fdiv_rn(amax, qmax) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const QuotientRounder qr(scale);
    const int quads_per_row = (cols + 3) / 4;
    const int chunks_per_row = (quads_per_row + kChunkQuads - 1) / kChunkQuads;
    const long long items = static_cast<long long>(chunks_per_row) * rows;
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
        const long long r = item / chunks_per_row;
        const int q0 = static_cast<int>(item - r * chunks_per_row) * kChunkQuads + static_cast<int>(threadIdx.x);
        const TIn* src_row = in + r * ld_in;
        uint8_t* dst_row = out + r * ld_out;
        if (vec_ok && (q0 + (U - 1) * kQuantThreads) * 4 + 4 <= cols) {
            typename Quad<TIn>::Raw v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = Quad<TIn>::load(src_row + (q0 + u * kQuantThreads) * 4);
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float x[4];
                Quad<TIn>::to_float(v[u], x);
                *reinterpret_cast<uint32_t*>(dst_row + (q0 + u * kQuantThreads) * 4) = quantize_quad<FP8>(x, qr);
            }
            continue;
        }
        for (int u = 0; u < U; ++u) {
            const int c = (q0 + u * kQuantThreads) * 4;
            if (c >= cols) break;
            if (vec_ok && c + 4 <= cols) {
                float x[4];
                Quad<TIn>::to_float(Quad<TIn>::load(src_row + c), x);
                *reinterpret_cast<uint32_t*>(dst_row + c) = quantize_quad<FP8>(x, qr);
            } else {
                for (int e = 0; e < 4 && c + e < cols; ++e)
                    dst_row[c + e] = quantize_one<FP8>(load_as_float(src_row + c + e), qr);
            }
        }
    }
}

// INT4 output: eight consecutive elements of a row become four packed bytes (one 32-bit store). Same (row, chunk)
// decomposition as quantize_kernel, a chunk being kQuantThreads x U groups of eight.
__device__ __forceinline__ uint32_t quantize_nibble(float x, const QuotientRounder& qr) {
    return qr.round_low_byte<7>(x) & 0xfu;
}

template <typename TIn>
__global__ void __launch_bounds__(kQuantThreads)
quantize_int4_kernel(const TIn* __restrict__ in, long long ld_in, uint8_t* __restrict__ out, long long ld_out_bytes,
                     int rows, int cols, const float* __restrict__ amax_in, float* __restrict__ scale_out, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    constexpr int U = Unroll<TIn>::value / 2;
    constexpr int kChunkOcts = kQuantThreads * U;
    const float amax = __ldg(amax_in);
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 7.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const QuotientRounder qr(scale);
    const int octs_per_row = (cols + 7) / 8;
    const int chunks_per_row = (octs_per_row + kChunkOcts - 1) / kChunkOcts;
    const long long items = static_cast<long long>(chunks_per_row) * rows;
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
        const long long r = item / chunks_per_row;
        const int o0 = static_cast<int>(item - r * chunks_per_row) * kChunkOcts + static_cast<int>(threadIdx.x);
        const TIn* src_row = in + r * ld_in;
        uint8_t* dst_row = out + r * ld_out_bytes;
        if (vec_ok && (o0 + (U - 1) * kQuantThreads) * 8 + 8 <= cols) {
            typename Quad<TIn>::Raw v[2 * U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                v[2 * u] = Quad<TIn>::load(src_row + (o0 + u * kQuantThreads) * 8);
                v[2 * u + 1] = Quad<TIn>::load(src_row + (o0 + u * kQuantThreads) * 8 + 4);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                float x[4], y[4];
                Quad<TIn>::to_float(v[2 * u], x);
                Quad<TIn>::to_float(v[2 * u + 1], y);
                uint32_t w = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    w |= quantize_nibble(x[e], qr) << (4 * e);
                    w |= quantize_nibble(y[e], qr) << (16 + 4 * e);
                }
                *reinterpret_cast<uint32_t*>(dst_row + (o0 + u * kQuantThreads) * 4) = w;
            }
            continue;
        }
        for (int u = 0; u < U; ++u) {
            const int c = (o0 + u * kQuantThreads) * 8;
            if (c >= cols) break;
            for (int e = 0; e < 8 && c + e < cols; e += 2) {  // cols is even: pairs are whole
                const uint32_t q0 = quantize_nibble(load_as_float(src_row + c + e), qr);
                const uint32_t q1 = quantize_nibble(load_as_float(src_row + c + e + 1), qr);
                dst_row[(c + e) >> 1] = static_cast<uint8_t>(q0 | (q1 << 4));
            }
        }
    }
}

__global__ void zero_float_kernel(float* p) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    *p = 0.0f;
}

template <typename TIn>
int quantize_typed(const TIn* in, size_t ld_in, void* out, size_t ld_out, float* scale_out, float* amax_out,
                   size_t rows, size_t cols, bool fp8, bool int4, int blocks, int vec_ok, cudaStream_t stream) {
    cudaError_t e = launch_pdl(zero_float_kernel, dim3(1), dim3(1), 0, stream, amax_out);
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;
    e = launch_pdl(amax_kernel<TIn>, dim3(blocks), dim3(kQuantThreads), 0, stream, in, (long long)ld_in, (int)rows,
                   (int)cols, amax_out, vec_ok);
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;
    if (int4)
        e = launch_pdl(quantize_int4_kernel<TIn>, dim3(blocks), dim3(kQuantThreads), 0, stream, in, (long long)ld_in,
                       static_cast<uint8_t*>(out), (long long)(ld_out / 2), (int)rows, (int)cols,
                       static_cast<const float*>(amax_out), scale_out, vec_ok);
    else if (fp8)
        e = launch_pdl(quantize_kernel<TIn, true>, dim3(blocks), dim3(kQuantThreads), 0, stream, in, (long long)ld_in,
                       static_cast<uint8_t*>(out), (long long)ld_out, (int)rows, (int)cols,
                       static_cast<const float*>(amax_out), scale_out, vec_ok);
    else
        e = launch_pdl(quantize_kernel<TIn, false>, dim3(blocks), dim3(kQuantThreads), 0, stream, in, (long long)ld_in,
                       static_cast<uint8_t*>(out), (long long)ld_out, (int)rows, (int)cols,
                       static_cast<const float*>(amax_out), scale_out, vec_ok);
    return e == cudaSuccess ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace

int quantize_launch(int in_dtype, int out_dtype, const void* in, size_t ld_in, void* out, size_t ld_out,
                    float* scale_out, float* amax_out, size_t rows, size_t cols, cudaStream_t stream) {
    if (in_dtype != QGEMM_DTYPE_FP32 && in_dtype != QGEMM_DTYPE_BF16) return QGEMM_ERR_UNSUPPORTED;
    if (out_dtype != QGEMM_DTYPE_FP8_E4M3 && out_dtype != QGEMM_DTYPE_INT8 && out_dtype != QGEMM_DTYPE_INT4)
        return QGEMM_ERR_UNSUPPORTED;
    const bool int4 = out_dtype == QGEMM_DTYPE_INT4;
    if (int4 && ((cols & 1) || (ld_out & 1))) return QGEMM_ERR_INVALID_ARG;
    if (scale_out == nullptr || amax_out == nullptr) return QGEMM_ERR_INVALID_ARG;
    if (rows > 0x7fffffffull || cols > 0x7fffffffull) return QGEMM_ERR_INVALID_ARG;
    if (rows > 0 && cols > 0 && (in == nullptr || out == nullptr || ld_in < cols || ld_out < cols))
        return QGEMM_ERR_INVALID_ARG;
    const size_t es = in_dtype == QGEMM_DTYPE_FP32 ? 4 : 2;
    // 4-element loads and 4-byte stores: for packed int4 output four bytes are eight elements
    const int vec_ok = (reinterpret_cast<uintptr_t>(in) % (4 * es) == 0) && (ld_in % 4 == 0) &&
                       (reinterpret_cast<uintptr_t>(out) % 4 == 0) && (ld_out % (int4 ? 8 : 4) == 0);
    // blocks walk (row, chunk) items: see amax_kernel
    const size_t chunk_quads = static_cast<size_t>(kQuantThreads) * (es == 4 ? 4 : 8);
    const size_t quads = (((cols + 3) / 4 + chunk_quads - 1) / chunk_quads) * rows * kQuantThreads;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    size_t blocks = (quads + kQuantThreads - 1) / kQuantThreads;
    blocks = blocks < 1 ? 1 : (blocks > static_cast<size_t>(sms) * 8 ? static_cast<size_t>(sms) * 8 : blocks);
    const bool fp8 = out_dtype == QGEMM_DTYPE_FP8_E4M3;
    if (in_dtype == QGEMM_DTYPE_FP32)
        return quantize_typed(static_cast<const float*>(in), ld_in, out, ld_out, scale_out, amax_out, rows, cols, fp8,
                              int4, static_cast<int>(blocks), vec_ok, stream);
    return quantize_typed(static_cast<const uint16_t*>(in), ld_in, out, ld_out, scale_out, amax_out, rows, cols, fp8,
                          int4, static_cast<int>(blocks), vec_ok, stream);
}

}  // namespace qgemm
