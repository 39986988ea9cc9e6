/*
 * CPU restatement of the QGEMM hot path -- TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker that the CUDA kernels are compared against. It is never part of
 * the shipped library: only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may load it.
 *
 * PARITY STATUS: the reference project ships no CPU GEMM, no golden vectors and no known-answer
 * tests for this path (its harness compares each kernel with cuBLAS at run time,
 * tests/includes/test_config.h:29-52,161-169). The arithmetic below restates the reference's
 * *semantics*, each function citing the reference lines it follows.
 *   - bf16 GEMM and transpose: PINNED. The reference's own GPU kernels (GEMM_kernel_v1/v2/v3/v3_1,
 *     matrix_transpose) were compiled from its sources (oracle/build_ref.sh) and run on a B200;
 *     their inputs and outputs are tests/golden/reference_bf16_gemm.npz and the CPU tests check
 *     this file against them.
 *   - int8 and FP8 mixed GEMM: parity unpinned -- the reference has no implementation of them for
 *     NVIDIA GPUs (src/mix_gemm/sm80_mix_gemm_kernel.cpp is empty) and none on the CPU. int8 is
 *     exact integer arithmetic; the FP8 conversions are checked against ml_dtypes and torch.
 *
 * Plain C99 + OpenMP; build with oracle/Makefile.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------------------------
 * Scalar format conversions.
 * -------------------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* fp32 -> bf16, round-to-nearest-even. The reference's helper adds 0x7fff + lsb to the bit
 * pattern and truncates (src/include/fast_quat.h:3-12) and has no NaN handling; this restatement
 * is the same rounding for every finite input and additionally keeps NaN a NaN. */
uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* fp32 -> IEEE binary16, round-to-nearest-even, overflow to infinity. */
uint16_t oracle_f32_to_f16(float f) {
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (abs >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);          /* >= 65520 -> inf */
    if (abs < 0x33000001u) return (uint16_t)sign;                       /* <= 2^-25 -> 0 */
    int32_t e = (int32_t)(abs >> 23) - 127;
    uint32_t m = (abs & 0x7fffffu) | 0x800000u;                          /* 24-bit significand */
    int shift;                                                           /* bits to drop */
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }                   /* subnormal half */
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));                                /* carry propagates into exponent */
}

float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    if (e == 0x1fu) return bits_f32(sign | 0x7f800000u | (m << 13));
    if (e == 0) {
        float v = (float)m * (1.0f / 16777216.0f);                      /* m * 2^-24 */
        return sign ? -v : v;
    }
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* OCP FP8 E4M3 ("e4m3fn": bias 7, max 448, no infinities, NaN = S.1111.111) as used by the CUDA
 * side of the reference (include/gpu_type.h:7, __nv_fp8_e4m3). */
float oracle_e4m3_to_f32(uint8_t b) {
    uint32_t sign = b >> 7;
    uint32_t e = (b >> 3) & 0xfu;
    uint32_t m = b & 7u;
    float v;
    if (e == 0xfu && m == 7u) return bits_f32(0x7fc00000u);
    if (e == 0) v = (float)m * (1.0f / 512.0f);                         /* m/8 * 2^-6 */
    else v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return sign ? -v : v;
}

/* fp32 -> e4m3fn, round-to-nearest-even with saturation to +-448 (the "satfinite" conversion). */
uint8_t oracle_f32_to_e4m3(float f) {
    uint32_t u = f32_bits(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t abs = u & 0x7fffffffu;
    if (abs > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
    float a = bits_f32(abs);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7eu);
    if (a < 0.0009765625f) return sign;                                 /* < 2^-10 rounds to 0 (tie at 2^-10 -> even = 0) */
    int e;
    (void)frexpf(a, &e);                                                /* a = frac * 2^e, frac in [0.5,1) */
    int exp = e - 1;                                                    /* a = 1.xxx * 2^exp */
    if (exp < -6) exp = -6;                                             /* subnormal range: fixed quantum 2^-9 */
    float quantum = ldexpf(1.0f, exp - 3);
    float q = a / quantum;                                              /* exact: power-of-two scaling */
    float r = rintf(q);                                                 /* ties-to-even in default rounding mode */
    float v = r * quantum;
    if (v > 448.0f) v = 448.0f;
    /* encode v */
    if (v == 0.0f) return sign;
    (void)frexpf(v, &e);
    exp = e - 1;
    if (exp < -6) {
        uint32_t m = (uint32_t)(v * 512.0f);
        return (uint8_t)(sign | m);
    }
    uint32_t m = (uint32_t)((v / ldexpf(1.0f, exp) - 1.0f) * 8.0f);
    return (uint8_t)(sign | ((uint32_t)(exp + 7) << 3) | m);
}

/* Vector forms used to prepare inputs. */
void oracle_round_bf16(const float* in, uint16_t* out_bits, float* out_f32, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint16_t b = oracle_f32_to_bf16(in[i]);
        if (out_bits) out_bits[i] = b;
        if (out_f32) out_f32[i] = oracle_bf16_to_f32(b);
    }
}

void oracle_round_f16(const float* in, uint16_t* out_bits, float* out_f32, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        uint16_t b = oracle_f32_to_f16(in[i]);
        if (out_bits) out_bits[i] = b;
        if (out_f32) out_f32[i] = oracle_f16_to_f32(b);
    }
}

/* Per-matrix FP8 quantisation: scale = amax / 448, q = e4m3(x / scale); the dequantised value is
 * scale * q. Returns the scale. */
float oracle_quantize_e4m3(const float* in, uint8_t* out_bits, float* out_f32, size_t n) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; ++i) { float a = fabsf(in[i]); if (a > amax) amax = a; }
    float scale = amax > 0.0f ? amax / 448.0f : 1.0f;
    for (size_t i = 0; i < n; ++i) {
        uint8_t b = oracle_f32_to_e4m3(in[i] / scale);
        if (out_bits) out_bits[i] = b;
        if (out_f32) out_f32[i] = oracle_e4m3_to_f32(b);
    }
    return scale;
}

/* Per-matrix int8 quantisation: scale = amax / 127, q = clamp(round_to_nearest_even(x / scale), -127, 127). */
float oracle_quantize_int8(const float* in, int8_t* out, size_t n) {
    float amax = 0.0f;
    for (size_t i = 0; i < n; ++i) { float a = fabsf(in[i]); if (a > amax) amax = a; }
    float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
    for (size_t i = 0; i < n; ++i) {
        float r = rintf(in[i] / scale);
        if (r > 127.0f) r = 127.0f;
        if (r < -127.0f) r = -127.0f;
        out[i] = (int8_t)(int)r;
    }
    return scale;
}

/* Packed signed 4-bit values (the roadmap's "Int4", develop.md:9-12; the reference has no code for it): two per
 * byte, element 2i in the low nibble of byte i, two's complement. */
void oracle_unpack_int4(const uint8_t* in, int8_t* out, size_t n_elems) {
    for (size_t i = 0; i < n_elems; ++i) {
        int nib = (i & 1) ? (in[i >> 1] >> 4) : (in[i >> 1] & 0x0f);
        out[i] = (int8_t)((nib ^ 8) - 8);
    }
}

/* Per-matrix int4 quantisation: scale = amax / 7, q = clamp(round_to_nearest_even(x / scale), -7, 7), packed as
 * above (n_elems even). Returns the scale. */
float oracle_quantize_int4(const float* in, uint8_t* out_packed, size_t n_elems) {
    float amax = 0.0f;
    for (size_t i = 0; i < n_elems; ++i) { float a = fabsf(in[i]); if (a > amax) amax = a; }
    float scale = amax > 0.0f ? amax / 7.0f : 1.0f;
    for (size_t i = 0; i < n_elems; i += 2) {
        int q[2];
        for (int e = 0; e < 2; ++e) {
            float r = rintf(in[i + e] / scale);
            if (r > 7.0f) r = 7.0f;
            if (r < -7.0f) r = -7.0f;
            q[e] = (int)r;
        }
        out_packed[i >> 1] = (uint8_t)((q[0] & 0xf) | ((q[1] & 0xf) << 4));
    }
    return scale;
}

void oracle_e4m3_decode(const uint8_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_e4m3_to_f32(in[i]);
}

void oracle_bf16_decode(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_bf16_to_f32(in[i]);
}

void oracle_f16_decode(const uint16_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) out[i] = oracle_f16_to_f32(in[i]);
}

/* ------------------------------------------------------------------------------------------
 * GEMM restatements.
 *
 * Layout (src/gemm/sm80_gemm_kernel_v1.cu:176-180 "All matrix are stored in row-major order"):
 *   A[m*lda + k]                        (src/include/gemm_utils.cuh:93)
 *   B[k*ldb + n]   when b_kmajor == 0   (src/include/gemm_utils.cuh:108)
 *   B[n*ldb + k]   when b_kmajor != 0   (src/include/gemm_utils.cuh:271, the v3.1/v4.1 operand form)
 *   C[m*ldc + n]                        (src/gemm/sm80_gemm_kernel_v1.cu:165-170)
 * Accumulators start at zero (src/gemm/sm80_gemm_kernel_v1.cu:128-135) and are fp32 for
 * floating inputs (cublasGemmEx compute type CUDA_R_32F, tests/includes/test_config.h:39-48) and
 * int32 for int8 inputs (src/gemm/test_cutlass_gemm.cu:68).
 * -------------------------------------------------------------------------------------- */

/* Floating GEMM on already-rounded inputs held as fp32; plain sequential-k fp32 accumulation. */
void oracle_gemm_f32(const float* A, size_t lda, const float* B, size_t ldb, int b_kmajor,
                     float* C, size_t ldc, size_t M, size_t N, size_t K) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t m = 0; m < (ptrdiff_t)M; ++m) {
        for (size_t n = 0; n < N; ++n) {
            float acc = 0.0f;
            if (b_kmajor) {
                const float* b = B + n * ldb;
                for (size_t k = 0; k < K; ++k) acc += A[m * lda + k] * b[k];
            } else {
                for (size_t k = 0; k < K; ++k) acc += A[m * lda + k] * B[k * ldb + n];
            }
            C[m * ldc + n] = acc;
        }
    }
}

/* The same product accumulated in fp64: the "truth" that both fp32 orders are measured against. */
void oracle_gemm_f64(const float* A, size_t lda, const float* B, size_t ldb, int b_kmajor,
                     double* C, size_t ldc, size_t M, size_t N, size_t K) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t m = 0; m < (ptrdiff_t)M; ++m) {
        for (size_t n = 0; n < N; ++n) {
            double acc = 0.0;
            if (b_kmajor) {
                const float* b = B + n * ldb;
                for (size_t k = 0; k < K; ++k) acc += (double)A[m * lda + k] * (double)b[k];
            } else {
                for (size_t k = 0; k < K; ++k) acc += (double)A[m * lda + k] * (double)B[k * ldb + n];
            }
            C[m * ldc + n] = acc;
        }
    }
}

/* int8 x int8 -> int32, exact (order-independent; |acc| <= K*127^2 fits for K <= 133000). */
void oracle_gemm_i8(const int8_t* A, size_t lda, const int8_t* B, size_t ldb, int b_kmajor,
                    int32_t* C, size_t ldc, size_t M, size_t N, size_t K) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t m = 0; m < (ptrdiff_t)M; ++m) {
        for (size_t n = 0; n < N; ++n) {
            int32_t acc = 0;
            if (b_kmajor) {
                const int8_t* b = B + n * ldb;
                for (size_t k = 0; k < K; ++k) acc += (int32_t)A[m * lda + k] * (int32_t)b[k];
            } else {
                for (size_t k = 0; k < K; ++k) acc += (int32_t)A[m * lda + k] * (int32_t)B[k * ldb + n];
            }
            C[m * ldc + n] = acc;
        }
    }
}

/* A row band [m0, m1) of the int8 product against K-major B: used to spot-check very large
 * problems without computing all of C. */
void oracle_gemm_i8_rows(const int8_t* A, size_t lda, const int8_t* B, size_t ldb,
                         int32_t* Cband, size_t ldc, size_t m0, size_t m1, size_t N, size_t K) {
#pragma omp parallel for schedule(static) collapse(2)
    for (ptrdiff_t m = (ptrdiff_t)m0; m < (ptrdiff_t)m1; ++m) {
        for (ptrdiff_t n = 0; n < (ptrdiff_t)N; ++n) {
            const int8_t* a = A + m * lda;
            const int8_t* b = B + n * ldb;
            int32_t acc = 0;
            for (size_t k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            Cband[(m - m0) * ldc + n] = acc;
        }
    }
}

/* Mixed-precision epilogue, C = (A o Q_A) x (B o Q_B) (README.md:5-7) with per-matrix scalar
 * coefficients: out = cast(sA * sB * acc). The scale product is formed in fp32 and applied to the
 * fp32 value of the accumulator, then rounded once to the output type, as the reference's only
 * mixed kernel does (src/mix_gemm/hip_mix_gemm_kernel.cpp:230-244 scale, :363-367 cast).
 * out_kind: 0 = fp32, 1 = bf16 bits, 2 = fp16 bits. */
void oracle_scale_cast_i32(const int32_t* acc, size_t n, float sA, float sB, int out_kind, void* out) {
    float alpha = sA * sB;
    for (size_t i = 0; i < n; ++i) {
        float v = alpha * (float)acc[i];
        if (out_kind == 0) ((float*)out)[i] = v;
        else if (out_kind == 1) ((uint16_t*)out)[i] = oracle_f32_to_bf16(v);
        else ((uint16_t*)out)[i] = oracle_f32_to_f16(v);
    }
}

void oracle_scale_cast_f32(const float* acc, size_t n, float sA, float sB, int out_kind, void* out) {
    float alpha = sA * sB;
    for (size_t i = 0; i < n; ++i) {
        float v = alpha * acc[i];
        if (out_kind == 0) ((float*)out)[i] = v;
        else if (out_kind == 1) ((uint16_t*)out)[i] = oracle_f32_to_bf16(v);
        else ((uint16_t*)out)[i] = oracle_f32_to_f16(v);
    }
}

/* Block-scaled FP8 GEMM, the one mixed kernel the reference implements
 * (src/mix_gemm/hip_mix_gemm_kernel.cpp:249-378). Operands are the decoded e4m3 values held as fp32:
 * A [M,K] row-major, Bt [N,K] (K-major). Scales as the reference lays them out (:124-169, :425-439):
 *   a_scale[kb*M + m]            one per row and 128-wide K block,
 *   b_scale[kb*ceil(N/128) + nb] one per 128 x 128 block of B.
 * Each K block is accumulated on its own in fp32 from zero and then folded in as
 * acc += local * a_scale * b_scale (:193-244); the result is rounded once to the output type
 * (:363-367). out_kind: 0 = fp32, 1 = bf16 bits, 2 = fp16 bits. */
void oracle_gemm_fp8_block_scaled(const float* A, size_t lda, const float* Bt, size_t ldb, const float* a_scale,
                                  const float* b_scale, void* C, size_t ldc, size_t M, size_t N, size_t K,
                                  int out_kind) {
    const size_t SB = 128;
    const size_t nbs = (N + SB - 1) / SB;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t m = 0; m < (ptrdiff_t)M; ++m) {
        for (size_t n = 0; n < N; ++n) {
            const float* a = A + m * lda;
            const float* b = Bt + n * ldb;
            float acc = 0.0f;
            for (size_t k0 = 0, kb = 0; k0 < K; k0 += SB, ++kb) {
                size_t k1 = k0 + SB < K ? k0 + SB : K;
                float local = 0.0f;
                for (size_t k = k0; k < k1; ++k) local += a[k] * b[k];
                acc += local * a_scale[kb * M + m] * b_scale[kb * nbs + n / SB];
            }
            if (out_kind == 0) ((float*)C)[m * ldc + n] = acc;
            else if (out_kind == 1) ((uint16_t*)C)[m * ldc + n] = oracle_f32_to_bf16(acc);
            else ((uint16_t*)C)[m * ldc + n] = oracle_f32_to_f16(acc);
        }
    }
}

/* Transpose: out[n*M + m] = in[m*N + n] (src/transpose/transpose.cu:42,57), any element size,
 * with explicit leading dimensions (in elements). */
void oracle_transpose(const void* in, void* out, size_t rows, size_t cols, size_t ld_in, size_t ld_out,
                      size_t elem_bytes) {
    const uint8_t* src = (const uint8_t*)in;
    uint8_t* dst = (uint8_t*)out;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)rows; ++r)
        for (size_t c = 0; c < cols; ++c)
            memcpy(dst + (c * ld_out + r) * elem_bytes, src + (r * ld_in + c) * elem_bytes, elem_bytes);
}

/* The reference harness's closed-form operand fill (tests/includes/test_config.h:251-258):
 * A[i] = (i % 43)/20 + 0.2 + (i % 19), B[i] = (i % 43)/20 + 0.2 + (i % 37), computed in double as
 * the C++ expression is, narrowed to float and then to the input type by the caller. */
void oracle_harness_fill(float* out, size_t n, int which_b) {
    for (size_t i = 0; i < n; ++i) {
        double v = (double)((float)(i % 43)) / 20.0 + 0.2 + (double)(i % (which_b ? 37 : 19));
        out[i] = (float)v;
    }
}

/* ------------------------------------------------------------------------------------------
 * Blocked, threaded forms of the same products: these are what the CPU baseline times. The
 * results equal the plain forms above exactly for int8 and up to fp32 summation order otherwise.
 * B must be K-major ([N,K]) so that both operands stream along k.
 * -------------------------------------------------------------------------------------- */

#define OR_BM 48
#define OR_BN 64
#define OR_BK 512

void oracle_gemm_f32_blocked(const float* A, size_t lda, const float* Bt, size_t ldb,
                             float* C, size_t ldc, size_t M, size_t N, size_t K) {
    size_t mt = (M + OR_BM - 1) / OR_BM, nt = (N + OR_BN - 1) / OR_BN;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (ptrdiff_t bm = 0; bm < (ptrdiff_t)mt; ++bm) {
        for (ptrdiff_t bn = 0; bn < (ptrdiff_t)nt; ++bn) {
            size_t m0 = bm * OR_BM, m1 = m0 + OR_BM < M ? m0 + OR_BM : M;
            size_t n0 = bn * OR_BN, n1 = n0 + OR_BN < N ? n0 + OR_BN : N;
            float acc[OR_BM][OR_BN];
            memset(acc, 0, sizeof(acc));
            for (size_t k0 = 0; k0 < K; k0 += OR_BK) {
                size_t k1 = k0 + OR_BK < K ? k0 + OR_BK : K;
                for (size_t m = m0; m < m1; ++m) {
                    const float* a = A + m * lda;
                    for (size_t n = n0; n < n1; ++n) {
                        const float* b = Bt + n * ldb;
                        float s = 0.0f;
#pragma omp simd reduction(+ : s)
                        for (size_t k = k0; k < k1; ++k) s += a[k] * b[k];
                        acc[m - m0][n - n0] += s;
                    }
                }
            }
            for (size_t m = m0; m < m1; ++m)
                for (size_t n = n0; n < n1; ++n) C[m * ldc + n] = acc[m - m0][n - n0];
        }
    }
}

void oracle_gemm_i8_blocked(const int8_t* A, size_t lda, const int8_t* Bt, size_t ldb,
                            int32_t* C, size_t ldc, size_t M, size_t N, size_t K) {
    size_t mt = (M + OR_BM - 1) / OR_BM, nt = (N + OR_BN - 1) / OR_BN;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (ptrdiff_t bm = 0; bm < (ptrdiff_t)mt; ++bm) {
        for (ptrdiff_t bn = 0; bn < (ptrdiff_t)nt; ++bn) {
            size_t m0 = bm * OR_BM, m1 = m0 + OR_BM < M ? m0 + OR_BM : M;
            size_t n0 = bn * OR_BN, n1 = n0 + OR_BN < N ? n0 + OR_BN : N;
            for (size_t m = m0; m < m1; ++m) {
                const int8_t* a = A + m * lda;
                for (size_t n = n0; n < n1; ++n) {
                    const int8_t* b = Bt + n * ldb;
                    int32_t s = 0;
#pragma omp simd reduction(+ : s)
                    for (size_t k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)b[k];
                    C[m * ldc + n] = s;
                }
            }
        }
    }
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
