// Declarations shared by the translation units of libqgemm.so (not installed).
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include <mutex>

#include "../../include/qgemm.h"

namespace qgemm {

int transpose_launch(const void* in, void* out, size_t rows, size_t cols, size_t ld_in, size_t ld_out,
                     size_t elem_bytes, cudaStream_t stream);

// Sums `splits` slabs of 32-bit partial accumulators (fp32, or int32 when acc_is_int) laid out as
// [split][M][ldw] and writes cast(scale_a*scale_b*sum) (out_kind: OUT_F32/BF16/F16) or the raw sum
// (OUT_RAW32) to C[M,N].
int splitk_reduce_launch(const void* partials, long long split_stride, long long ldw, int splits, bool acc_is_int,
                         void* C, long long ldc, int M, int N, int out_kind, const float* scale_a,
                         const float* scale_b, cudaStream_t stream);

// Per-matrix quantisation: amax reduction, scale = amax / qmax, out = round(in / scale) (quantize.cu).
int quantize_launch(int in_dtype, int out_dtype, const void* in, size_t ld_in, void* out, size_t ld_out,
                    float* scale_out, float* amax_out, size_t rows, size_t cols, cudaStream_t stream);

// Widens packed signed 4-bit values (two per byte, low nibble first) to int8: out[r*ld_out + c] for c < cols.
// ld_in_elems counts 4-bit elements (even); cols even (int4.cu).
int unpack_int4_launch(const void* in, size_t ld_in_elems, void* out, size_t ld_out, size_t rows, size_t cols,
                       cudaStream_t stream);

// The one lock of the dispatch layer: the per-device scratch, the tensor-map cache and the per-device "kernel
// attributes configured" flags of the launchers are only touched while it is held (capi.cu).
std::mutex& dispatch_mutex();

// The K block armed by qgemm_test_arm_skip_load (-1 = none); disarms. Called with the dispatch lock held by the
// launch that consumes it.
int take_test_skip_kb();

// QGEMM_* environment variables, read when the library is loaded and again by qgemm_reload_env().
struct EnvSettings {
    int tile_n = 0, split_k = 0, group_m = 0, cta_pair = 0, relayout_b = 0, max_ctas = 0, direct_store = 0;
    int full_a_tile = 0, tail_split_off = 0, balance = 0, prefetch_off = 0, prefetch_force = 0, kcluster_off = 0, kcluster_pair_off = 0, kgroup = 0, early_groups = -1, one_tile_off = 0, even_runs = 0;
    int host_bands = 0, host_bands_n = 0;  // 0 = default
};
const EnvSettings& env_settings();

// Status words of the allocation-free entry point on the current device: copied to host4 and cleared when they
// record an error; all zero when that entry point has not been used on this device. Allocates nothing (no_alloc.cu).
int static_status_fetch(int host4[4]);

// Frees the streams, events and device buffers of the host-operand path (host_gemm.cu).
void host_path_shutdown();

}  // namespace qgemm
