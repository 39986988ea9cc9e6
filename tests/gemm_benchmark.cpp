// C++ benchmark harness for the library, in the shape of the reference's unfinished
// tests/gemm_benchmark.cpp skeleton (struct TestConfig, class GemmTestFramework, calculate_tflops,
// a results table; tests/gemm_benchmark.cpp:14-163 of the reference, which does not compile) and with
// the row format of its working harness (tests/includes/test_config.h:137-159), so the reference's
// scripts/benchmark_to_md.py parses this program's output unchanged:
//
//   Problem size: M=..., N=..., K=...
//   <function> <time ms> <TFLOPS> <GB/s> <PASS|FAIL> <max error> <speedup vs vendor>
//
// It calls the library only through the C++ templates of include/gemm.h (device pointers, default
// stream), times with CUDA events like the reference (warm-up runs, then back-to-back timed runs), uses
// cublasGemmEx as the vendor row for the 16-bit precisions exactly as the reference harness does
// (tests/includes/test_config.h:29-52), and checks every kernel against a host computation of sampled
// output rows (fp32 / int32 dot products on the same rounded inputs).
//
// Build:  nvcc -std=c++17 -O2 -I include tests/gemm_benchmark.cpp -L qgemm_b200 -lqgemm -lcublas -o tests/gemm_benchmark
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <functional>
#include <iomanip>
#include <iostream>
#include <string>
#include <type_traits>
#include <vector>

#include "blas.h"
#include "gemm.h"
#include "matrix_transpose.h"

struct TestConfig {
    int M, N, K;
    std::string precision;  // "bf16", "fp16", "int8", "fp8"
    int warmup_runs;
    int benchmark_runs;
    TestConfig(int m, int n, int k, const std::string& prec = "bf16", int warmup = 2, int bench = 5)
        : M(m), N(n), K(k), precision(prec), warmup_runs(warmup), benchmark_runs(bench) {}
};

namespace {

#define CHECK_CUDA(x)                                                                         \
    do {                                                                                      \
        cudaError_t e_ = (x);                                                                 \
        if (e_ != cudaSuccess) {                                                              \
            std::cerr << "CUDA error " << cudaGetErrorString(e_) << " at " << #x << std::endl; \
            std::exit(2);                                                                     \
        }                                                                                     \
    } while (0)

// Deterministic operand values in [-1, 1): a 64-bit mix of (seed, index).
inline float unit_value(uint64_t seed, uint64_t i) {
    uint64_t z = (seed + 0x9e3779b97f4a7c15ull) ^ (i * 0xbf58476d1ce4e5b9ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return static_cast<float>(static_cast<double>(z >> 11) / 9007199254740992.0 * 2.0 - 1.0);
}

template <typename T> struct Conv;
template <> struct Conv<__nv_bfloat16> {
    static __nv_bfloat16 from(float f) { return __float2bfloat16(f); }
    static float to(__nv_bfloat16 v) { return __bfloat162float(v); }
};
template <> struct Conv<__half> {
    static __half from(float f) { return __float2half(f); }
    static float to(__half v) { return __half2float(v); }
};
template <> struct Conv<int8_t> {
    static int8_t from(float f) { return static_cast<int8_t>(std::lrintf(f * 127.0f)); }
    static float to(int8_t v) { return static_cast<float>(v); }
};
template <> struct Conv<__nv_fp8_e4m3> {
    static __nv_fp8_e4m3 from(float f) { return __nv_fp8_e4m3(f * 4.0f); }
    static float to(__nv_fp8_e4m3 v) { return static_cast<float>(v); }
};
template <> struct Conv<float> {
    static float to(float v) { return v; }
};
template <> struct Conv<int32_t> {
    static float to(int32_t v) { return static_cast<float>(v); }
};

double time_ms(const std::function<void()>& fn, int warmup, int runs) {
    for (int i = 0; i < warmup; ++i) fn();
    cudaEvent_t a, b;
    CHECK_CUDA(cudaEventCreate(&a));
    CHECK_CUDA(cudaEventCreate(&b));
    CHECK_CUDA(cudaEventRecord(a));
    for (int i = 0; i < runs; ++i) fn();
    CHECK_CUDA(cudaEventRecord(b));
    CHECK_CUDA(cudaEventSynchronize(b));
    float ms = 0.f;
    CHECK_CUDA(cudaEventElapsedTime(&ms, a, b));
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return ms / runs;
}

}  // namespace

class GemmTestFramework {
public:
    GemmTestFramework() { blas::blas_init(blas_handle_); }
    ~GemmTestFramework() { blas::blas_destroy(blas_handle_); }

    double calculate_tflops(const TestConfig& config, double ms) const {
        return 2.0 * config.M * config.N * config.K / (ms / 1000.0) / 1e12;
    }

    void print_results(const std::string& name, const TestConfig& c, double ms, size_t elem_bytes, bool pass,
                       double max_err, double vendor_ms) const {
        const double gbs = (double(c.M) * c.K + double(c.K) * c.N + double(c.M) * c.N) * elem_bytes / (ms * 1e-3) / 1e9;
        std::cout << std::left << std::setw(28) << name << std::fixed << std::setprecision(4) << std::setw(12) << ms
                  << std::setprecision(2) << std::setw(12) << calculate_tflops(c, ms) << std::setw(15) << gbs
                  << std::setw(12) << (pass ? "PASS" : "FAIL") << std::scientific << std::setprecision(2)
                  << std::setw(16) << max_err << std::setw(16) << (vendor_ms > 0 ? vendor_ms / ms : 1.0) << std::endl;
        if (!pass) ++failures_;
    }

    // One configuration of precision TIn -> TOut; `mixed` = scaled mixed-precision entry point.
    template <typename TIn, typename TOut, bool mixed>
    void run_config(const TestConfig& c, double tol_rel) {
        const size_t M = c.M, N = c.N, K = c.K;
        std::vector<TIn> hA(M * K), hB(K * N);
        for (size_t i = 0; i < hA.size(); ++i) hA[i] = Conv<TIn>::from(unit_value(1, i));
        for (size_t i = 0; i < hB.size(); ++i) hB[i] = Conv<TIn>::from(unit_value(2, i));
        TIn *dA, *dB;
        TOut* dC;
        float* dS;
        CHECK_CUDA(cudaMalloc(&dA, hA.size() * sizeof(TIn)));
        CHECK_CUDA(cudaMalloc(&dB, hB.size() * sizeof(TIn)));
        CHECK_CUDA(cudaMalloc(&dC, M * N * sizeof(TOut)));
        CHECK_CUDA(cudaMalloc(&dS, 2 * sizeof(float)));
        CHECK_CUDA(cudaMemcpy(dA, hA.data(), hA.size() * sizeof(TIn), cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(TIn), cudaMemcpyHostToDevice));
        const float hS[2] = {0.0078125f, 0.015625f};
        CHECK_CUDA(cudaMemcpy(dS, hS, sizeof(hS), cudaMemcpyHostToDevice));
        const float alpha = mixed ? hS[0] * hS[1] : 1.0f;

        std::cout << "\n=== GEMM Benchmark ===\nProblem size: M=" << M << ", N=" << N << ", K=" << K
                  << "\nPrecision: " << c.precision << "\nWarmup runs: " << c.warmup_runs
                  << "\nBenchmark runs: " << c.benchmark_runs << "\n" << std::string(110, '=') << "\n"
                  << std::left << std::setw(28) << "Function" << std::setw(12) << "Time(ms)" << std::setw(12) << "TFLOPS"
                  << std::setw(15) << "Bandwidth(GB/s)" << std::setw(12) << "Correctness" << std::setw(16)
                  << "Max Error" << std::setw(16) << "Speedup" << "\n" << std::string(110, '-') << std::endl;

        double vendor_ms = -1.0;
        if constexpr (std::is_same_v<TIn, __nv_bfloat16> || std::is_same_v<TIn, __half>) {
            const cudaDataType in_t = std::is_same_v<TIn, __half> ? CUDA_R_16F : CUDA_R_16BF;
            const cudaDataType out_t = std::is_same_v<TOut, float> ? CUDA_R_32F : in_t;
            const float one = 1.0f, zero = 0.0f;
            auto vendor = [&]() {  // row-major C = A x B through the operand swap the reference uses
                cublasGemmEx(blas_handle_, CUBLAS_OP_N, CUBLAS_OP_N, (int)N, (int)M, (int)K, &one, dB, in_t, (int)N, dA,
                             in_t, (int)K, &zero, dC, out_t, (int)N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
            };
            vendor_ms = time_ms(vendor, c.warmup_runs, c.benchmark_runs);
            CHECK_CUDA(cudaDeviceSynchronize());
            auto chk = check(hA, hB, dC, M, N, K, 1.0f, tol_rel);
            print_results("reference_cublas", c, vendor_ms, sizeof(TIn), chk.first, chk.second, vendor_ms);
        }

        auto run_and_report = [&](const std::string& name, const std::function<void()>& fn) {
            CHECK_CUDA(cudaMemset(dC, 0, M * N * sizeof(TOut)));
            const double ms = time_ms(fn, c.warmup_runs, c.benchmark_runs);
            CHECK_CUDA(cudaDeviceSynchronize());
            const bool ok_status = qgemm_last_status() == QGEMM_OK;
            auto chk = check(hA, hB, dC, M, N, K, alpha, tol_rel);
            print_results(name, c, ms, sizeof(TIn), chk.first && ok_status, chk.second, vendor_ms);
        };
        if constexpr (mixed) {
            run_and_report("MIX_GEMM_kernel", [&]() { MIX_GEMM_kernel<TIn, TOut>(dA, K, dB, N, dS, dS + 1, dC, N, M, N, K); });
        } else {
            run_and_report("GEMM_kernel_v1", [&]() { GEMM_kernel_v1<TIn, TOut>(dA, K, dB, N, dC, N, M, N, K); });
            run_and_report("GEMM_kernel_v5", [&]() { GEMM_kernel_v5<TIn, TOut>(dA, K, dB, N, dC, N, M, N, K); });
        }
        std::cout << std::string(110, '=') << std::endl;
        cudaFree(dA);
        cudaFree(dB);
        cudaFree(dC);
        cudaFree(dS);
    }

    // matrix_transpose<T> against a host transpose (exact).
    template <typename T>
    void run_transpose(int rows, int cols, const std::string& name) {
        std::vector<T> h(size_t(rows) * cols), back(size_t(rows) * cols);
        for (size_t i = 0; i < h.size(); ++i) h[i] = Conv<T>::from(unit_value(3, i));
        T *din, *dout;
        CHECK_CUDA(cudaMalloc(&din, h.size() * sizeof(T)));
        CHECK_CUDA(cudaMalloc(&dout, h.size() * sizeof(T)));
        CHECK_CUDA(cudaMemcpy(din, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
        const double ms = time_ms([&]() { matrix_transpose<T>(din, dout, rows, cols); }, 2, 10);
        CHECK_CUDA(cudaMemcpy(back.data(), dout, h.size() * sizeof(T), cudaMemcpyDeviceToHost));
        size_t bad = 0;
        for (int r = 0; r < rows; r += 7)
            for (int c = 0; c < cols; ++c)
                bad += std::memcmp(&back[size_t(c) * rows + r], &h[size_t(r) * cols + c], sizeof(T)) != 0;
        const double gbs = 2.0 * h.size() * sizeof(T) / (ms * 1e-3) / 1e9;
        std::cout << "matrix_transpose<" << name << "> " << rows << "x" << cols << ": " << std::fixed
                  << std::setprecision(4) << ms << " ms, " << std::setprecision(0) << gbs << " GB/s, "
                  << (bad == 0 ? "PASS" : "FAIL") << std::endl;
        if (bad) ++failures_;
        cudaFree(din);
        cudaFree(dout);
    }

    // The shape presets of the reference's tests/includes/example_configs.h:8-53 -- "small", "medium", "large" and
    // "mixed" (square, tall, wide and two transformer projection shapes), with its warm-up / run counts -- for one
    // precision. An unknown name gives an empty list.
    static std::vector<TestConfig> preset(const std::string& name, const std::string& precision) {
        struct Row { int m, n, k, warmup, runs; };
        std::vector<Row> rows;
        if (name == "small") rows = {{128, 128, 128, 3, 10}, {256, 256, 256, 3, 10}, {512, 512, 512, 3, 10}};
        else if (name == "medium") rows = {{512, 512, 512, 5, 20}, {1024, 1024, 1024, 5, 20}, {2048, 2048, 2048, 5, 20}};
        else if (name == "large") rows = {{2048, 2048, 2048, 3, 10}, {4096, 4096, 4096, 3, 10}, {8192, 8192, 8192, 3, 5}};
        else if (name == "mixed")
            rows = {{512, 512, 512, 5, 10},   {1024, 1024, 1024, 5, 10}, {2048, 512, 1024, 5, 10},  {4096, 1024, 2048, 5, 10},
                    {512, 2048, 1024, 5, 10}, {1024, 4096, 2048, 5, 10}, {1024, 4096, 1024, 5, 10}, {4096, 1024, 4096, 5, 10}};
        std::vector<TestConfig> out;
        for (const Row& r : rows) out.emplace_back(r.m, r.n, r.k, precision, r.warmup, r.runs);
        return out;
    }

    void run_benchmark(const std::string& preset_name = "", const std::string& precision = "bf16") {
        std::cout << "\n=== QGEMM Benchmark Results ===" << std::endl;
        std::vector<TestConfig> configs = {
            TestConfig(1024, 1024, 1024, "fp16"), TestConfig(1024, 1024, 1024, "bf16"),
            TestConfig(2048, 2048, 2048, "bf16"), TestConfig(4096, 4096, 4096, "bf16"),
            TestConfig(1000, 1016, 520, "bf16"),  TestConfig(4096, 4096, 4096, "int8"),
            TestConfig(4096, 4096, 4096, "fp8"),  TestConfig(64, 7168, 2048, "fp8"),
        };
        if (!preset_name.empty()) configs = preset(preset_name, precision);
        for (const auto& c : configs) {
            if (c.precision == "bf16") run_config<__nv_bfloat16, float, false>(c, 1e-3);
            else if (c.precision == "fp16") run_config<__half, float, false>(c, 1e-3);
            else if (c.precision == "int8") {
                run_config<int8_t, int32_t, false>(c, 0.0);
                run_config<int8_t, __nv_bfloat16, true>(c, 8e-3);
            } else run_config<__nv_fp8_e4m3, __nv_bfloat16, true>(c, 1e-2);
        }
        std::cout << std::endl;
        if (!preset_name.empty()) return;
        run_transpose<__nv_bfloat16>(8192, 8192, "bf16");
        run_transpose<int8_t>(4096, 8192, "int8");
        run_transpose<__nv_bfloat16>(1000, 333, "bf16");
    }

    int failures() const { return failures_; }

private:
    // Host check of sampled rows: |c - ref| <= tol_rel * max(|ref|, rms of the row) (exact when tol_rel == 0).
    template <typename TIn, typename TOut>
    std::pair<bool, double> check(const std::vector<TIn>& hA, const std::vector<TIn>& hB, const TOut* dC, size_t M,
                                  size_t N, size_t K, float alpha, double tol_rel) {
        std::vector<TOut> hC(M * N);
        CHECK_CUDA(cudaMemcpy(hC.data(), dC, hC.size() * sizeof(TOut), cudaMemcpyDeviceToHost));
        std::vector<float> bcol(K);
        double max_err = 0.0;
        bool ok = true;
        const size_t rows[4] = {0, M / 3, (2 * M) / 3 + 1 < M ? (2 * M) / 3 + 1 : M - 1, M - 1};
        std::vector<double> ref(N);
        for (size_t ri = 0; ri < 4; ++ri) {
            const size_t m = rows[ri];
            std::fill(ref.begin(), ref.end(), 0.0);
            for (size_t k = 0; k < K; ++k) {
                const double a = Conv<TIn>::to(hA[m * K + k]);
                for (size_t n = 0; n < N; ++n) ref[n] += a * Conv<TIn>::to(hB[k * N + n]);
            }
            double ss = 0.0;
            for (size_t n = 0; n < N; ++n) { ref[n] *= alpha; ss += ref[n] * ref[n]; }
            const double rms = std::sqrt(ss / N);
            for (size_t n = 0; n < N; ++n) {
                const double err = std::fabs(double(Conv<TOut>::to(hC[m * N + n])) - ref[n]);
                max_err = std::max(max_err, err);
                if (err > tol_rel * std::max(std::fabs(ref[n]), rms)) ok = false;
            }
        }
        return {ok, max_err};
    }

    blas_handle_t blas_handle_ = nullptr;
    mutable int failures_ = 0;
};

// gemm_benchmark                      the library's own shape list, every precision, then the transposes
// gemm_benchmark <preset> [precision] one of the reference's presets: small | medium | large | mixed; precision
//                                     bf16 (default) | fp16 | int8 | fp8
int main(int argc, char** argv) {
    const std::string preset_name = argc > 1 ? argv[1] : "";
    const std::string precision = argc > 2 ? argv[2] : "bf16";
    if (!preset_name.empty() && GemmTestFramework::preset(preset_name, precision).empty()) {
        std::cerr << "unknown preset '" << preset_name << "' (small | medium | large | mixed)" << std::endl;
        return 2;
    }
    if (precision != "bf16" && precision != "fp16" && precision != "int8" && precision != "fp8") {
        std::cerr << "unknown precision '" << precision << "' (bf16 | fp16 | int8 | fp8)" << std::endl;
        return 2;
    }
    std::cout << "QGEMM Benchmark Test Suite" << std::endl;
    cudaDeviceProp prop;
    CHECK_CUDA(cudaGetDeviceProperties(&prop, 0));
    std::cout << "GPU: " << prop.name << "\nCompute Capability: " << prop.major << "." << prop.minor << std::endl;
    GemmTestFramework framework;
    framework.run_benchmark(preset_name, precision);
    if (framework.failures() != 0) {
        std::cout << "\n" << framework.failures() << " check(s) FAILED" << std::endl;
        return 1;
    }
    std::cout << "\nBenchmark completed successfully!" << std::endl;
    return 0;
}
