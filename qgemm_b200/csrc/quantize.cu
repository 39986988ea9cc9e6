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

// One thread handles 4 consecutive elements of a row; quads_per_row = ceil(cols / 4).
template <typename TIn>
__global__ void __launch_bounds__(kQuantThreads)
amax_kernel(const TIn* __restrict__ in, long long ld, int rows, int cols, float* __restrict__ amax_out, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const long long quads_per_row = (cols + 3) / 4;
    const long long total = quads_per_row * rows;
    float m = 0.0f;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / quads_per_row;
        const int c = static_cast<int>(i - r * quads_per_row) * 4;
        const TIn* src = in + r * ld + c;
        if (vec_ok && c + 4 <= cols) {
            if constexpr (sizeof(TIn) == 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(src));
                m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            } else {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
                m = fmaxf(m, fmaxf(fmaxf(fabsf(__low2float(a)), fabsf(__high2float(a))),
                                   fmaxf(fabsf(__low2float(b)), fabsf(__high2float(b)))));
            }
        } else {
            for (int e = 0; e < 4 && c + e < cols; ++e) m = fmaxf(m, fabsf(load_as_float(src + e)));
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

template <bool FP8>
__device__ __forceinline__ uint8_t quantize_one(float x, float scale) {
    const float q = __fdiv_rn(x, scale);
    if constexpr (FP8) {
        return static_cast<uint8_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3));
    } else {
        const float r = fminf(fmaxf(rintf(q), -127.0f), 127.0f);
        return static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(r)));
    }
}

template <typename TIn, bool FP8>
__global__ void __launch_bounds__(kQuantThreads)
quantize_kernel(const TIn* __restrict__ in, long long ld_in, uint8_t* __restrict__ out, long long ld_out, int rows,
                int cols, const float* __restrict__ amax_in, float* __restrict__ scale_out, int vec_ok) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const float amax = __ldg(amax_in);
    const float qmax = FP8 ? 448.0f : 127.0f;
    const float scale = amax > 0.0f ? __fdiv_rn(amax, qmax) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const long long quads_per_row = (cols + 3) / 4;
    const long long total = quads_per_row * rows;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / quads_per_row;
        const int c = static_cast<int>(i - r * quads_per_row) * 4;
        const TIn* src = in + r * ld_in + c;
        uint8_t* dst = out + r * ld_out + c;
        if (vec_ok && c + 4 <= cols) {
            float x[4];
            if constexpr (sizeof(TIn) == 4) {
                const float4 v = __ldg(reinterpret_cast<const float4*>(src));
                x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
            } else {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
                x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
            }
            const uint32_t packed = quantize_one<FP8>(x[0], scale) | (quantize_one<FP8>(x[1], scale) << 8) |
                                    (quantize_one<FP8>(x[2], scale) << 16) |
                                    (static_cast<uint32_t>(quantize_one<FP8>(x[3], scale)) << 24);
            *reinterpret_cast<uint32_t*>(dst) = packed;
        } else {
            for (int e = 0; e < 4 && c + e < cols; ++e) dst[e] = quantize_one<FP8>(load_as_float(src + e), scale);
        }
    }
}

// INT4 output: one thread handles 8 consecutive elements of a row and writes 4 packed bytes.
template <typename TIn>
__global__ void __launch_bounds__(kQuantThreads)
quantize_int4_kernel(const TIn* __restrict__ in, long long ld_in, uint8_t* __restrict__ out, long long ld_out_bytes,
                     int rows, int cols, const float* __restrict__ amax_in, float* __restrict__ scale_out) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const float amax = __ldg(amax_in);
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 7.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
    const long long octs_per_row = (cols + 7) / 8;
    const long long total = octs_per_row * rows;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long r = i / octs_per_row;
        const int c = static_cast<int>(i - r * octs_per_row) * 8;
        const TIn* src = in + r * ld_in + c;
        uint8_t* dst = out + r * ld_out_bytes + c / 2;
        for (int e = 0; e < 8 && c + e < cols; e += 2) {  // cols is even: pairs are whole
            const float q0 = fminf(fmaxf(rintf(__fdiv_rn(load_as_float(src + e), scale)), -7.0f), 7.0f);
            const float q1 = fminf(fmaxf(rintf(__fdiv_rn(load_as_float(src + e + 1), scale)), -7.0f), 7.0f);
            dst[e >> 1] = static_cast<uint8_t>((static_cast<int>(q0) & 0xf) | ((static_cast<int>(q1) & 0xf) << 4));
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
                       static_cast<const float*>(amax_out), scale_out);
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
    const int vec_ok = (reinterpret_cast<uintptr_t>(in) % (4 * es) == 0) && (ld_in % 4 == 0) &&
                       (reinterpret_cast<uintptr_t>(out) % 4 == 0) && (ld_out % 4 == 0);
    const size_t quads = ((cols + 3) / 4) * rows;
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
