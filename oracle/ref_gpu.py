"""Loader for oracle/_ref/libqgemm_ref.so -- the reference project's OWN GPU kernels, compiled
unmodified from its source tree by oracle/build_ref.sh (compute_89 PTX, JIT-compiled on the B200).

TEST INFRASTRUCTURE ONLY: it exists to pin the CPU oracle (and through it the CUDA kernels) to
what the reference itself computes. It is never part of the shipped path.

The reference kernels have no bounds checks and a tile-grouping clamp that is only right for whole
groups (src/gemm/sm80_gemm_kernel_v1.cu:104-117), so `check_shape` admits only shapes every one of
them handles: M % 512 == 0, N % 128 == 0, K % 64 == 0.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libqgemm_ref.so")

# Itanium-mangled names of the explicit specialisations <__nv_bfloat16, float>
# (e.g. src/gemm/sm89_gemm_kernel_v3.cu:311-324) and of matrix_transpose<__nv_bfloat16>
# (src/transpose/transpose.cu:76).
_GEMM_SYMBOLS = {
    "v1": "_Z14GEMM_kernel_v1I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
    "v2": "_Z14GEMM_kernel_v2I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
    "v3": "_Z14GEMM_kernel_v3I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
    "v3_1": "_Z16GEMM_kernel_v3_1I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",  # consumes B as [N,K]
    "v4": "_Z14GEMM_kernel_v4I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
}
_TRANSPOSE_SYMBOL = "_Z16matrix_transposeI13__nv_bfloat16EvPKT_PS1_ii"

_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
    return _lib


def check_shape(M: int, N: int, K: int) -> None:
    if M % 512 or N % 128 or K % 64 or min(M, N, K) <= 0:
        raise ValueError("reference kernels need M % 512 == 0, N % 128 == 0, K % 64 == 0")


def launcher(version: str):
    """The raw entry point GEMM_kernel_<version><bf16,float>(A, ldA, B, ldB, C, ldC, M, N, K) (legacy default
    stream, asynchronous), for timing loops. Shapes must satisfy check_shape."""
    fn = getattr(lib(), _GEMM_SYMBOLS[version])
    fn.restype = None
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                   C.c_size_t]
    return fn


def gemm(version: str, a, b, c) -> None:
    """Run the reference's GEMM_kernel_<version><bf16,float> on torch CUDA tensors (default stream).
    a [M,K] bf16; b [K,N] bf16 (or [N,K] for v3_1); c [M,N] fp32, all contiguous."""
    import torch
    M, K = a.shape
    N = c.shape[1]
    check_shape(M, N, K)
    assert a.is_contiguous() and b.is_contiguous() and c.is_contiguous()
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and c.dtype == torch.float32
    fn = getattr(lib(), _GEMM_SYMBOLS[version])
    fn.restype = None
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                   C.c_size_t]
    torch.cuda.current_stream().synchronize()  # the reference launches on the legacy default stream
    fn(a.data_ptr(), K, b.data_ptr(), b.shape[1], c.data_ptr(), N, M, N, K)
    torch.cuda.synchronize()


def transpose(x, out) -> None:
    """Reference matrix_transpose<bf16>(in [M,N]) -> out [N,M]; needs M % 64 == 0 and N % 32 == 0."""
    import torch
    M, N = x.shape
    if M % 64 or N % 32:
        raise ValueError("reference transpose needs M % 64 == 0 and N % 32 == 0")
    assert x.is_contiguous() and out.is_contiguous() and x.dtype == torch.bfloat16
    fn = getattr(lib(), _TRANSPOSE_SYMBOL)
    fn.restype = None
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
    torch.cuda.current_stream().synchronize()
    fn(x.data_ptr(), out.data_ptr(), M, N)
    torch.cuda.synchronize()
