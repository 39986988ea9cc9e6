// Sharing an output buffer between the processes of one box, for qgemm_gemm_multi_dst.
//
// The column-sharded GEMM runs one process per GPU; to let every rank's epilogue store its block of C
// straight into every other rank's full matrix, each rank exports the device allocation that holds its
// matrix and maps the others'. This file is that plumbing and nothing else: CUDA's inter-process memory
// handles (64 opaque bytes that any transport can carry), the offset of the buffer inside its allocation,
// and the matching open / close. The reference has nothing multi-GPU (every launch on the default stream of
// one device, e.g. src/gemm/sm80_gemm_kernel_v4.cu:344-349), so none of this replaces reference code.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>

#include "qgemm_internal.h"

namespace {

using AddressRangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);

AddressRangeFn address_range_fn() {
    static AddressRangeFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<AddressRangeFn>(p);
    }
    return fn;
}

}  // namespace

extern "C" {

int qgemm_peer_export(const void* ptr, void* handle_out, size_t* offset_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == QGEMM_PEER_HANDLE_BYTES, "handle size");
    if (ptr == nullptr || handle_out == nullptr || offset_out == nullptr) return QGEMM_ERR_INVALID_ARG;
    AddressRangeFn range = address_range_fn();
    if (range == nullptr) return QGEMM_ERR_CUDA;
    // make sure the primary context is current before the driver call
    if (cudaFree(nullptr) != cudaSuccess) return QGEMM_ERR_CUDA;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return QGEMM_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_CUDA;
    }
    std::memcpy(handle_out, &h, sizeof(h));
    *offset_out = static_cast<size_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
    return QGEMM_OK;
}

int qgemm_peer_alloc(size_t bytes, void** ptr_out) {
    if (ptr_out == nullptr || bytes == 0) return QGEMM_ERR_INVALID_ARG;
    void* p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_WORKSPACE;
    }
    *ptr_out = p;
    return QGEMM_OK;
}

int qgemm_peer_free(void* ptr) {
    if (ptr == nullptr) return QGEMM_OK;
    if (cudaFree(ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_CUDA;
    }
    return QGEMM_OK;
}

int qgemm_peer_open(const void* handle, void** base_out) {
    if (handle == nullptr || base_out == nullptr) return QGEMM_ERR_INVALID_ARG;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* base = nullptr;
    if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_CUDA;
    }
    *base_out = base;
    return QGEMM_OK;
}

int qgemm_peer_close(void* base) {
    if (base == nullptr) return QGEMM_OK;
    if (cudaIpcCloseMemHandle(base) != cudaSuccess) {
        (void)cudaGetLastError();
        return QGEMM_ERR_CUDA;
    }
    return QGEMM_OK;
}

}  // extern "C"
