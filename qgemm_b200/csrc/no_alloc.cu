// qgemm_mix_gemm_splitk_static: the split-K GEMM for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a GEMM: real-time
// loops that forbid anything that may synchronise the whole device, embedders whose memory budget
// is fixed at start-up, and processes where another allocator already owns all of the GPU's memory
// so that an allocation made by this library would simply fail. The ordinary split-K path keeps
// its partial sums in a scratch buffer that the library grows with cudaMalloc; this entry point
// keeps them in a fixed array that is part of the loaded module instead, so it never allocates,
// frees or grows anything -- on the device or through any allocating library routine.
//
// The price is a fixed cap (QGEMM_STATIC_SCRATCH_BYTES, reserved on every GPU that loads the library
// until the process exits) and a shared buffer: every call on a device uses the same array, which
// still holds the previous call's partial sums. Nothing in it needs to start at zero -- the GEMM pass
// overwrites every partial the reduction pass reads for the rows and columns it writes -- but two
// calls that overlap on the GPU (for example on different streams with no ordering) race on it.
//
// A bounded wait that runs out in this path is recorded in status words that are part of the module as well;
// qgemm_device_status reads and clears them (static_status_fetch below) without allocating.
//
// The first call on a device does the set-up (cudaGetSymbolAddress for the two arrays, the kernel's
// shared-memory attribute); it should come before any stream capture is started.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>

#include "gemm_launch.cuh"
#include "qgemm_internal.h"

namespace qgemm {
namespace {

// The scratch itself and the status words of this path. In host code these names are host-side
// stand-ins, not device addresses: the addresses handed to kernels come from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[QGEMM_STATIC_SCRATCH_BYTES];
static __device__ __align__(256) int g_static_status[16];

constexpr int kMaxDevicesStatic = 64;

struct StaticDevice {
    bool ready = false;
    void* scratch = nullptr;  // device address of g_static_scratch on this device
    int* status = nullptr;    // device address of g_static_status on this device
    int sm_count = 0;
};

StaticDevice g_static_dev[kMaxDevicesStatic];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_static_encode = nullptr;

// One-time set-up of the current device: resolves the device addresses of the static arrays.
int static_setup(StaticDevice** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevicesStatic) return QGEMM_ERR_UNSUPPORTED;
    StaticDevice& s = g_static_dev[dev];
    if (!s.ready) {
        int cc_major = 0;
        if (cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return QGEMM_ERR_CUDA;
        if (cc_major != 10) return QGEMM_ERR_UNSUPPORTED;
        if (cudaDeviceGetAttribute(&s.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            return QGEMM_ERR_CUDA;
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return QGEMM_ERR_CUDA;
        s.scratch = p;
        void* st = nullptr;
        if (cudaGetSymbolAddress(&st, g_static_status) != cudaSuccess || st == nullptr) return QGEMM_ERR_CUDA;
        s.status = static_cast<int*>(st);
        s.ready = true;
    }
    if (g_static_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || fn == nullptr)
            return QGEMM_ERR_CUDA;
        g_static_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = &s;
    return QGEMM_OK;
}

int encode_operand(const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, int in_dtype, uint32_t box_rows,
                   CUtensorMap* out) {
    CUtensorMapDataType dt;
    uint32_t es;
    switch (in_dtype) {
        case QGEMM_DTYPE_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; es = 2; break;
        case QGEMM_DTYPE_FP16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; es = 2; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; es = 1; break;
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {ld * es};
    const cuuint32_t box[2] = {128u / es, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_static_encode(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QGEMM_OK : QGEMM_ERR_CUDA;
}

// [splits][M][ldw] 32-bit partial sums in the static scratch, for the kernel's TMA-store epilogue.
int encode_partials(void* ptr, uint64_t M, uint64_t N, uint64_t ldw, uint64_t splits, CUtensorMap* out) {
    const cuuint64_t dims[3] = {N, M, splits};
    const cuuint64_t strides[2] = {ldw * 4, M * ldw * 4};
    const cuuint32_t box[3] = {32u, 32u, 1u};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = g_static_encode(out, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, ptr, dims, strides, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? QGEMM_OK : QGEMM_ERR_CUDA;
}

}  // namespace

// Called by qgemm_device_status with the dispatch lock held and the device synchronised.
int static_status_fetch(int host4[4]) {
    host4[0] = host4[1] = host4[2] = host4[3] = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevicesStatic || !g_static_dev[dev].ready) return QGEMM_OK;
    int* words = g_static_dev[dev].status;
    if (cudaMemcpy(host4, words, 4 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return QGEMM_ERR_CUDA;
    if (host4[0] != 0 && cudaMemset(words, 0, 4 * sizeof(int)) != cudaSuccess) return QGEMM_ERR_CUDA;
    return QGEMM_OK;
}

}  // namespace qgemm

using namespace qgemm;

extern "C" int qgemm_mix_gemm_splitk_static(int in_dtype, int out_dtype, const void* A, size_t lda, const void* B,
                                            size_t ldb, const float* scale_a, const float* scale_b, void* C,
                                            size_t ldc, size_t M, size_t N, size_t K, int split_k,
                                            qgemm_stream_t stream) {
    if (M == 0 || N == 0) return QGEMM_OK;
    if (A == nullptr || B == nullptr || C == nullptr || K == 0) return QGEMM_ERR_INVALID_ARG;
    if (lda < K || ldb < K || ldc < N || split_k < 2) return QGEMM_ERR_INVALID_ARG;
    if (M > 0x7fffff00ull || N > 0x7fffff00ull || K > 0x7fffff00ull) return QGEMM_ERR_INVALID_ARG;

    int kind, es;
    uint32_t fmt, cfmt;
    bool acc_int = false;
    switch (in_dtype) {
        case QGEMM_DTYPE_BF16: kind = ptx::KIND_F16; es = 2; fmt = 1; cfmt = 1; break;
        case QGEMM_DTYPE_FP16: kind = ptx::KIND_F16; es = 2; fmt = 0; cfmt = 1; break;
        case QGEMM_DTYPE_INT8: kind = ptx::KIND_I8; es = 1; fmt = 1; cfmt = 2; acc_int = true; break;
        case QGEMM_DTYPE_FP8_E4M3: kind = ptx::KIND_F8; es = 1; fmt = 0; cfmt = 1; break;
        default: return QGEMM_ERR_UNSUPPORTED;
    }
    int out_kind;
    switch (out_dtype) {
        case QGEMM_DTYPE_FP32: out_kind = OUT_F32; break;
        case QGEMM_DTYPE_BF16: out_kind = OUT_BF16; break;
        case QGEMM_DTYPE_FP16: out_kind = OUT_F16; break;
        case QGEMM_DTYPE_INT32: out_kind = OUT_RAW32; break;
        default: return QGEMM_ERR_UNSUPPORTED;
    }
    if (out_kind == OUT_RAW32 && (!acc_int || scale_a != nullptr || scale_b != nullptr)) return QGEMM_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(A) % 16 != 0 || (lda * es) % 16 != 0) return QGEMM_ERR_ALIGNMENT;
    if (reinterpret_cast<uintptr_t>(B) % 16 != 0 || (ldb * es) % 16 != 0) return QGEMM_ERR_ALIGNMENT;

    // Same plan the allocating path makes for tile_n = 128 and this split count.
    constexpr int kTileN = 128;
    const int kblk = 128 / es;
    const int kb_total = static_cast<int>((K + kblk - 1) / kblk);
    if (split_k > kb_total) return QGEMM_ERR_INVALID_ARG;
    const int kb_per_split = (kb_total + split_k - 1) / split_k;
    const int splits = (kb_total + kb_per_split - 1) / kb_per_split;
    const size_t ldw = (N + 3) / 4 * 4;
    const size_t need = static_cast<size_t>(splits) * M * ldw * 4;
    if (need > static_cast<size_t>(QGEMM_STATIC_SCRATCH_BYTES)) return QGEMM_ERR_WORKSPACE;  // beyond the fixed cap

    std::lock_guard<std::mutex> lock(dispatch_mutex());
    StaticDevice* st = nullptr;
    int rc = static_setup(&st);
    if (rc != QGEMM_OK) return rc;

    CUtensorMap ta, tb;
    rc = encode_operand(A, M, K, lda, in_dtype, kBM, &ta);
    if (rc != QGEMM_OK) return rc;
    rc = encode_operand(B, N, K, ldb, in_dtype, kTileN, &tb);
    if (rc != QGEMM_OK) return rc;

    CUtensorMap tc;
    rc = encode_partials(st->scratch, M, N, ldw, static_cast<uint64_t>(splits), &tc);
    if (rc != QGEMM_OK) return rc;

    GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.C = st->scratch;
    p.ldc = static_cast<long long>(ldw);
    p.split_stride = static_cast<long long>(M) * static_cast<long long>(ldw);
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.m_tiles = static_cast<int>((M + kBM - 1) / kBM);
    p.n_tiles = static_cast<int>((N + kTileN - 1) / kTileN);
    p.splits = splits;
    p.kb_total = kb_total;
    p.kb_per_split = kb_per_split;
    p.group_m = 8;
    p.idesc = ptx::make_idesc(cfmt, fmt, fmt, kBM, kTileN);
    p.status = st->status;
    p.c_vec_ok = 1;
    p.c_tma_ok = 1;
    p.test_skip_kb = take_test_skip_kb();

    const long long work = static_cast<long long>(p.m_tiles) * p.n_tiles * p.splits;
    if (work > 0x7fffffffLL) return QGEMM_ERR_UNSUPPORTED;
    const int grid = static_cast<int>(work < st->sm_count ? work : st->sm_count);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e;
    switch (kind) {
        case ptx::KIND_F16: e = launch_gemm_f16(kTileN, OUT_RAW32, kBM, ta, tb, tc, p, grid, s); break;
        case ptx::KIND_I8: e = launch_gemm_i8(kTileN, OUT_RAW32, kBM, ta, tb, tc, p, grid, s); break;
        default: e = launch_gemm_f8(kTileN, OUT_RAW32, kBM, ta, tb, tc, p, grid, s); break;
    }
    if (e != cudaSuccess) return QGEMM_ERR_CUDA;
    return splitk_reduce_launch(st->scratch, p.split_stride, p.ldc, splits, acc_int, C, static_cast<long long>(ldc),
                                p.M, p.N, out_kind, scale_a, scale_b, s);
}
