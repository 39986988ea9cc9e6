/*! \file blas.h
 *  \brief Handle lifecycle with the names the reference harness calls
 *  (include/blas.h:19-50: blas::blas_handle, blas::blas_init, blas::blas_destroy; used at
 *  tests/includes/test_config.h:208,298). The handle is a cuBLAS handle because the harness passes
 *  blas::blas_handle to cublasGemmEx for its own reference result (tests/includes/test_config.h:39).
 *
 *  Differences from the reference header: everything is `inline` (the reference defines non-inline
 *  functions and a global in a header, which breaks when two translation units include it), there
 *  is no CUTLASS include, and blas_destroy() also releases this library's per-device scratch.
 */
#pragma once
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include "qgemm.h"

using blas_handle_t = cublasHandle_t;

namespace blas {

inline blas_handle_t blas_handle = nullptr;

inline void blas_init(blas_handle_t& handle) { cublasCreate(&handle); }
inline void blas_init() { blas_init(blas_handle); }

inline void blas_destroy(blas_handle_t& handle) {
    if (handle != nullptr) cublasDestroy(handle);
    handle = nullptr;
    qgemm_shutdown();
}
inline void blas_destroy() { blas_destroy(blas_handle); }

}  // namespace blas
