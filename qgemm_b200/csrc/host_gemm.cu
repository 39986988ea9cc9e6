// qgemm_gemm_host: C = A x B with all three matrices in HOST memory.
//
// This is the flow of the reference's own harness -- allocate on the host, copy to the device, run the
// kernel, copy C back (tests/includes/test_config.h:239-286) -- done as one call and as a pipeline. The
// PCIe link is the bound (three matrices cross it, the product itself takes a tenth of that time), so the
// point is to keep the upload engine busy from the first byte to the last and to have as little as possible
// left to do after the last byte arrives:
//   * B is uploaded in column bands and A in row bands, alternately, so that the set of (row band, column
//     band) blocks of C whose operands are both on the device grows like a square. Every arriving band is
//     followed by ONE GEMM over all blocks it completes (a row strip or a column strip of C) and by the
//     download of that strip, on a second copy engine, while later bands are still uploading. The first
//     block of C is on its way back after 1/8 of A and 1/8 of B, instead of after all of B.
//   * The last row bands of A are halved repeatedly down to 256 rows, and B is complete before them: what remains
//     after the final upload is the GEMM and download of a thin strip of whole rows of C (contiguous in host memory;
//     column strips move in short runs and reach 37 GB/s where row strips reach 46-50).
// All device work goes through qgemm_gemm_ex (the ordinary kernels); nothing here computes.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "qgemm_internal.h"

namespace qgemm {

namespace {

constexpr int kMaxDev = 64;
constexpr int kEventPool = 256;
constexpr int kDefaultBands = 8;

struct HostPath {
    bool init = false;
    cudaStream_t s_in = nullptr, s_compute = nullptr, s_out = nullptr;
    cudaEvent_t ev[kEventPool] = {};
    int next_ev = 0;
    cudaEvent_t ev_prev_done = nullptr;  // completion of the previous call: its device buffers are free again
    bool have_prev = false;
    void* arena = nullptr;  // [A | B | C | two scale floats]
    size_t arena_bytes = 0;
};

std::mutex g_host_mutex;
HostPath g_host[kMaxDev];

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t elem_bytes_of(int dtype) {
    switch (dtype) {
        case QGEMM_DTYPE_BF16:
        case QGEMM_DTYPE_FP16: return 2;
        case QGEMM_DTYPE_INT8:
        case QGEMM_DTYPE_FP8_E4M3: return 1;
        case QGEMM_DTYPE_FP32:
        case QGEMM_DTYPE_INT32: return 4;
        default: return 0;
    }
}

struct Band {
    size_t lo, hi;
};

// About `bands` equal bands of whole 256-row tiles; with `shrink`, the last of them halved down to 256.
std::vector<Band> band_schedule(size_t extent, int bands, bool shrink) {
    std::vector<Band> out;
    if (extent == 0) return out;
    bands = std::max(1, bands);
    size_t rows = (extent + bands - 1) / bands;
    rows = round_up(rows, 256);
    std::vector<size_t> sizes;
    for (size_t left = extent; left > 0;) {
        const size_t s = std::min(rows, left);
        sizes.push_back(s);
        left -= s;
    }
    size_t last = sizes.back();
    sizes.pop_back();
    while (shrink && last > 256) {
        const size_t half = round_up(last / 2, 256);
        if (half >= last) break;
        sizes.push_back(half);
        last -= half;
    }
    sizes.push_back(last);
    size_t r = 0;
    for (size_t s : sizes) {
        out.push_back({r, r + s});
        r += s;
    }
    return out;
}

int ensure_host_path(HostPath& h, size_t arena_bytes) {
    if (!h.init) {
        if (cudaStreamCreateWithFlags(&h.s_in, cudaStreamNonBlocking) != cudaSuccess) return QGEMM_ERR_CUDA;
        if (cudaStreamCreateWithFlags(&h.s_compute, cudaStreamNonBlocking) != cudaSuccess) return QGEMM_ERR_CUDA;
        if (cudaStreamCreateWithFlags(&h.s_out, cudaStreamNonBlocking) != cudaSuccess) return QGEMM_ERR_CUDA;
        for (int i = 0; i < kEventPool; ++i)
            if (cudaEventCreateWithFlags(&h.ev[i], cudaEventDisableTiming) != cudaSuccess) return QGEMM_ERR_CUDA;
        if (cudaEventCreateWithFlags(&h.ev_prev_done, cudaEventDisableTiming) != cudaSuccess) return QGEMM_ERR_CUDA;
        h.init = true;
    }
    if (arena_bytes > h.arena_bytes) {
        // earlier calls may still be using the old buffers
        if (cudaDeviceSynchronize() != cudaSuccess) return QGEMM_ERR_CUDA;
        if (h.arena) cudaFree(h.arena);
        h.arena = nullptr;
        h.arena_bytes = 0;
        const size_t rounded = round_up(arena_bytes, (size_t)1 << 20);
        if (cudaMalloc(&h.arena, rounded) != cudaSuccess) {
            (void)cudaGetLastError();
            return QGEMM_ERR_WORKSPACE;
        }
        h.arena_bytes = rounded;
    }
    return QGEMM_OK;
}

#define QG_CUDA(call)                                  \
    do {                                               \
        if ((call) != cudaSuccess) {                   \
            (void)cudaGetLastError();                  \
            return QGEMM_ERR_CUDA;                     \
        }                                              \
    } while (0)

cudaEvent_t next_event(HostPath& h) {
    cudaEvent_t e = h.ev[h.next_ev];
    h.next_ev = (h.next_ev + 1) % kEventPool;
    return e;
}

}  // namespace

void host_path_shutdown() {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    int cur = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) return;
    for (int d = 0; d < kMaxDev; ++d) {
        HostPath& h = g_host[d];
        if (!h.init && h.arena == nullptr) continue;
        cudaSetDevice(d);
        cudaDeviceSynchronize();
        if (h.arena) cudaFree(h.arena);
        if (h.init) {
            cudaStreamDestroy(h.s_in);
            cudaStreamDestroy(h.s_compute);
            cudaStreamDestroy(h.s_out);
            for (int i = 0; i < kEventPool; ++i) cudaEventDestroy(h.ev[i]);
            cudaEventDestroy(h.ev_prev_done);
        }
        h = HostPath();
    }
    cudaSetDevice(cur);
}

}  // namespace qgemm

using namespace qgemm;

extern "C" int qgemm_host_band_schedule(size_t extent, int bands, int shrink, size_t* edges_out, int max_bands) {
    const std::vector<Band> b = band_schedule(extent, bands > 0 ? bands : kDefaultBands, shrink != 0);
    const int n = static_cast<int>(b.size());
    if (edges_out != nullptr)
        for (int i = 0; i < n && i < max_bands; ++i) {
            edges_out[2 * i] = b[i].lo;
            edges_out[2 * i + 1] = b[i].hi;
        }
    return n;
}

namespace {

// A_dev != nullptr: A is already on the device (leading dimension lda, 16-byte aligned rows) and only B is uploaded;
// every arriving column band of B is followed by the GEMM and download of the column strip of C it completes.
int host_gemm_impl(int in_dtype, int out_dtype, int b_layout, const void* A_host, const void* A_dev, size_t lda,
                   const void* B_host, size_t ldb, const float* scale_a_host, const float* scale_b_host,
                   void* C_host, size_t ldc, size_t M, size_t N, size_t K, cudaStream_t stream) {
    const bool a_resident = A_dev != nullptr;
    if (a_resident) A_host = A_dev;  // only tested against null below
    const size_t es = elem_bytes_of(in_dtype), os = elem_bytes_of(out_dtype);
    if (es == 0 || es > 2 || os < 2) return QGEMM_ERR_UNSUPPORTED;
    if (b_layout != QGEMM_B_ROW_MAJOR && b_layout != QGEMM_B_K_MAJOR) return QGEMM_ERR_INVALID_ARG;
    if (M == 0 || N == 0) return QGEMM_OK;
    if (C_host == nullptr || ldc < N) return QGEMM_ERR_INVALID_ARG;
    const bool kmajor = b_layout == QGEMM_B_K_MAJOR;
    if (K > 0 && (A_host == nullptr || B_host == nullptr || lda < K || ldb < (kmajor ? K : N)))
        return QGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return QGEMM_ERR_INVALID_ARG;

    int dev = 0;
    QG_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDev) return QGEMM_ERR_UNSUPPORTED;

    // Device copies with tight, 16-byte-aligned leading dimensions.
    const size_t align_in = 16 / es, align_out = 16 / os;
    const size_t lda_d = round_up(std::max<size_t>(K, 1), align_in);
    const size_t ldb_d = kmajor ? lda_d : round_up(N, align_in);
    const size_t ldc_d = round_up(N, align_out);
    const size_t a_bytes = a_resident ? 0 : round_up(M * lda_d * es, 256);
    const size_t b_bytes = round_up((kmajor ? N : std::max<size_t>(K, 1)) * ldb_d * es, 256);
    const size_t c_bytes = round_up(M * ldc_d * os, 256);

    std::lock_guard<std::mutex> lock(g_host_mutex);
    HostPath& h = g_host[dev];
    int rc = ensure_host_path(h, a_bytes + b_bytes + c_bytes + 256);
    if (rc != QGEMM_OK) return rc;
    const uint8_t* a_d = a_resident ? static_cast<const uint8_t*>(A_dev) : static_cast<uint8_t*>(h.arena);
    const size_t lda_use = a_resident ? lda : lda_d;
    uint8_t* b_d = static_cast<uint8_t*>(h.arena) + a_bytes;
    uint8_t* c_d = b_d + b_bytes;
    float* scales_d = reinterpret_cast<float*>(c_d + c_bytes);

    // Everything below is ordered after the caller's stream and after the previous call on this device.
    cudaEvent_t ev_start = next_event(h);
    QG_CUDA(cudaEventRecord(ev_start, stream));
    for (cudaStream_t s : {h.s_in, h.s_compute, h.s_out}) {
        QG_CUDA(cudaStreamWaitEvent(s, ev_start, 0));
        if (h.have_prev) QG_CUDA(cudaStreamWaitEvent(s, h.ev_prev_done, 0));
    }

    const float* sa_d = nullptr;
    const float* sb_d = nullptr;
    if (scale_a_host != nullptr) {
        QG_CUDA(cudaMemcpyAsync(scales_d, scale_a_host, sizeof(float), cudaMemcpyHostToDevice, h.s_in));
        sa_d = scales_d;
    }
    if (scale_b_host != nullptr) {
        QG_CUDA(cudaMemcpyAsync(scales_d + 1, scale_b_host, sizeof(float), cudaMemcpyHostToDevice, h.s_in));
        sb_d = scales_d + 1;
    }

    const EnvSettings& env = env_settings();
    const int want_bands = env.host_bands > 0 ? env.host_bands : kDefaultBands;
    const int want_bands_n = env.host_bands_n > 0 ? env.host_bands_n : want_bands;
    // Only the row bands shrink towards the end: the strips that are left after the last byte has arrived should be
    // whole rows of C (contiguous in host memory), not narrow column blocks.
    std::vector<Band> mb = band_schedule(M, want_bands, true);
    std::vector<Band> nb = band_schedule(N, want_bands_n, false);
    if (K == 0) {  // nothing to upload: one strip, C = 0
        mb.assign(1, Band{0, M});
        nb.assign(1, Band{0, N});
    }
    if (a_resident) mb.clear();

    // One GEMM over the strip C[r0:r1, c0:c1] and its download.
    auto strip = [&](size_t r0, size_t r1, size_t c0, size_t c1, cudaEvent_t operands_ready) -> int {
        QG_CUDA(cudaStreamWaitEvent(h.s_compute, operands_ready, 0));
        const uint8_t* b_ptr = kmajor ? b_d + c0 * ldb_d * es : b_d + c0 * es;
        const int g = qgemm_gemm_ex(in_dtype, out_dtype, b_layout, a_d + r0 * lda_use * es, lda_use, b_ptr, ldb_d, sa_d, sb_d,
                                    c_d + (r0 * ldc_d + c0) * os, ldc_d, r1 - r0, c1 - c0, K, nullptr, h.s_compute);
        if (g != QGEMM_OK) return g;
        cudaEvent_t done = next_event(h);
        QG_CUDA(cudaEventRecord(done, h.s_compute));
        QG_CUDA(cudaStreamWaitEvent(h.s_out, done, 0));
        QG_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(C_host) + (r0 * ldc + c0) * os, ldc * os,
                                  c_d + (r0 * ldc_d + c0) * os, ldc_d * os, (c1 - c0) * os, r1 - r0,
                                  cudaMemcpyDeviceToHost, h.s_out));
        return QGEMM_OK;
    };

    size_t rows_up = a_resident ? M : 0, cols_up = 0;  // rows of A and columns of B that are on the device
    size_t ia = 0, ib = 0;
    while (ia < mb.size() || ib < nb.size()) {
        // alternate, B first, keeping the loaded part of C close to square; B is complete before the last, thin row
        // bands of A, so that the final strips are row strips
        const bool take_a = ib >= nb.size() || (ia < mb.size() && rows_up * N < cols_up * M);
        if (take_a) {
            const Band b = mb[ia++];
            if (K > 0)
                QG_CUDA(cudaMemcpy2DAsync(static_cast<uint8_t*>(h.arena) + b.lo * lda_d * es, lda_d * es,
                                          static_cast<const uint8_t*>(A_host) + b.lo * lda * es, lda * es, K * es,
                                          b.hi - b.lo, cudaMemcpyHostToDevice, h.s_in));
            cudaEvent_t up = next_event(h);
            QG_CUDA(cudaEventRecord(up, h.s_in));
            rows_up = b.hi;
            if (cols_up > 0) {
                rc = strip(b.lo, b.hi, 0, cols_up, up);
                if (rc != QGEMM_OK) return rc;
            }
        } else {
            const Band b = nb[ib++];
            if (K > 0) {
                if (kmajor)
                    QG_CUDA(cudaMemcpy2DAsync(b_d + b.lo * ldb_d * es, ldb_d * es,
                                              static_cast<const uint8_t*>(B_host) + b.lo * ldb * es, ldb * es, K * es,
                                              b.hi - b.lo, cudaMemcpyHostToDevice, h.s_in));
                else
                    QG_CUDA(cudaMemcpy2DAsync(b_d + b.lo * es, ldb_d * es,
                                              static_cast<const uint8_t*>(B_host) + b.lo * es, ldb * es,
                                              (b.hi - b.lo) * es, K, cudaMemcpyHostToDevice, h.s_in));
            }
            cudaEvent_t up = next_event(h);
            QG_CUDA(cudaEventRecord(up, h.s_in));
            cols_up = b.hi;
            if (rows_up > 0) {
                rc = strip(0, rows_up, b.lo, b.hi, up);
                if (rc != QGEMM_OK) return rc;
            }
        }
    }

    // The caller's stream continues once all three legs are done; so does the next call's use of the buffers.
    for (cudaStream_t s : {h.s_in, h.s_compute, h.s_out}) {
        cudaEvent_t e = next_event(h);
        QG_CUDA(cudaEventRecord(e, s));
        QG_CUDA(cudaStreamWaitEvent(stream, e, 0));
    }
    QG_CUDA(cudaEventRecord(h.ev_prev_done, stream));
    h.have_prev = true;
    return QGEMM_OK;
}

}  // namespace

extern "C" int qgemm_gemm_host(int in_dtype, int out_dtype, int b_layout, const void* A_host, size_t lda,
                               const void* B_host, size_t ldb, const float* scale_a_host, const float* scale_b_host,
                               void* C_host, size_t ldc, size_t M, size_t N, size_t K, qgemm_stream_t stream) {
    return host_gemm_impl(in_dtype, out_dtype, b_layout, A_host, nullptr, lda, B_host, ldb, scale_a_host, scale_b_host,
                          C_host, ldc, M, N, K, static_cast<cudaStream_t>(stream));
}

extern "C" int qgemm_gemm_host_resident_a(int in_dtype, int out_dtype, int b_layout, const void* A_dev, size_t lda,
                                          const void* B_host, size_t ldb, const float* scale_a_host,
                                          const float* scale_b_host, void* C_host, size_t ldc, size_t M, size_t N,
                                          size_t K, qgemm_stream_t stream) {
    if (A_dev == nullptr) return QGEMM_ERR_INVALID_ARG;
    return host_gemm_impl(in_dtype, out_dtype, b_layout, nullptr, A_dev, lda, B_host, ldb, scale_a_host, scale_b_host,
                          C_host, ldc, M, N, K, static_cast<cudaStream_t>(stream));
}
