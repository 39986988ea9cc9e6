/*! \file gemm.h
 *  \brief C++ API of the B200 quantized-GEMM library: same function-template names, argument order
 *  and meaning as the reference's include/gemm.h:25-66, implemented on top of the C-ABI in qgemm.h.
 *
 *  All pointers are device pointers; all matrices are row-major with explicit leading dimensions
 *  in elements ("All matrix are stored in row-major order", src/gemm/sm80_gemm_kernel_v1.cu:176-180).
 *  Calls enqueue work on the default stream and return without synchronising, as the reference's
 *  do. Errors are reported the way the reference reports them -- a message on std::cerr and a
 *  void return (src/gemm/sm80_gemm_kernel_v3.cu:295-299) -- and additionally kept for
 *  qgemm_last_status().
 *
 *  The definitions live in libqgemm.so as explicit specialisations for the type pairs listed at
 *  the end of this file; link against it instead of the reference's gemm_lib.
 */
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "qgemm.h"

/* ---- C = A x B, B given as [K,N] row-major (include/gemm.h:25-66) ------------------------------
 * GEMM_kernel_v1 ... v5 were successive optimisation steps of one operation in the reference; here
 * every name runs the same sm_100a kernel. (The reference's v3_1 / v4_1 silently reinterpret B as
 * [N,K] while their caller passes [K,N], src/gemm/sm80_gemm_kernel_v3.1.cu:292; that defect is not
 * reproduced: use GEMM_kernel_kmajor for a K-major B.)
 * Specialised for <__nv_bfloat16|__half, float|__nv_bfloat16|__half> and <int8_t, int32_t>. */
template <typename typeIn, typename typeOut>
void GEMM_kernel_v1(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                    size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v2(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                    size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v3(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                    size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v3_1(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                      size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v4(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                    size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v4_1(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                      size_t N, size_t K);
template <typename typeIn, typename typeOut>
void GEMM_kernel_v5(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                    size_t N, size_t K);

/* ---- C = A x B with B K-major: B[n*ldB + k] ("col-major [K,N]"), the operand form the reference's
 * v3_1 / v4_1 loaders consume (src/include/gemm_utils.cuh:263-273). No relayout pass is needed. */
template <typename typeIn, typename typeOut>
void GEMM_kernel_kmajor(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M,
                        size_t N, size_t K);

/* ---- Mixed precision C = (A o Q_A) x (B o Q_B) (README.md:5-7), per-matrix scalar coefficients.
 * Argument order follows the reference's (a, b, as, bs, c) entry points
 * (src/mix_gemm/hip_mix_gemm_kernel.cpp:508-516). scaleA / scaleB are device pointers to one float.
 * B is [K,N] row-major for MIX_GEMM_kernel and K-major ([N,K], as fp8_mm takes it) for
 * MIX_GEMM_kernel_kmajor. Specialised for <int8_t|__nv_fp8_e4m3, __nv_bfloat16|__half|float>. */
template <typename typeIn, typename typeOut>
void MIX_GEMM_kernel(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, const float* scaleA,
                     const float* scaleB, typeOut* C, size_t ldC, size_t M, size_t N, size_t K);
template <typename typeIn, typename typeOut>
void MIX_GEMM_kernel_kmajor(const typeIn* A, size_t ldA, const typeIn* B, size_t ldB, const float* scaleA,
                            const float* scaleB, typeOut* C, size_t ldC, size_t M, size_t N, size_t K);

/* ---- Vendor-baseline entry points the reference harness links against (include/gemm.h:11-22,
 * used at tests/cuda_benchmark.cpp:63-75). The reference implements them with CUTLASS 2.x /
 * cuBLAS (third-party libraries, out of scope here); these symbols run the library's own kernel
 * so that an unmodified harness links and its table rows stay meaningful.
 * Specialised for <__nv_bfloat16,float>, <__nv_bfloat16,__nv_bfloat16> and <int8_t,int8_t>
 * (int8 output saturates the int32 accumulator to [-128,127] as the vendor kernels do). */
template <typename typeIn, typename typeOut>
void cutlass_gemm_test(typeIn* A, size_t ldA, typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M, size_t N,
                       size_t K);
template <typename typeIn, typename typeOut>
void cublas_gemm_test(typeIn* A, size_t ldA, typeIn* B, size_t ldB, typeOut* C, size_t ldC, size_t M, size_t N,
                      size_t K);

/* Status of the most recent call made through this header on the calling thread (a qgemm_status_t). */
int qgemm_last_status();
