"""GEMM on HOST operands: the call a user of the reference harness effectively makes -- host
buffers in, host result out (tests/includes/test_config.h:239-286 allocates on the host, copies to
the device, runs the kernel and copies C back).

``HostGemm`` is a thin wrapper over the C-ABI entry ``qgemm_gemm_host``, which owns the device
buffers and overlaps the three legs itself: B goes up in column bands and A in row bands,
alternately, each arriving band is followed by one GEMM over the blocks of C it completes and by
their download while later bands are still uploading, so a step costs about the upload time plus a
thin last strip instead of upload + GEMM + download. Nothing here computes or copies.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import B_K_MAJOR, B_ROW_MAJOR, QgemmError, ERR_INVALID_ARG, _check, _dtype_code, lib


def band_schedule(extent: int, bands: int = 8, shrink: bool = True):
    """The bands [lo, hi) ``qgemm_gemm_host`` cuts an extent into, as the library itself computes them
    (``qgemm_host_band_schedule``): about ``bands`` equal ones made of whole 256-wide tiles; with ``shrink`` (the
    rows of A) the last of them is halved repeatedly down to 256, so that what is left after the final upload is a
    thin strip's GEMM and download. The columns of B are cut without it."""
    if extent <= 0:
        return []
    L = lib()
    n = L.qgemm_host_band_schedule(int(extent), int(bands), 1 if shrink else 0, None, 0)
    buf = (C.c_size_t * (2 * n))()
    L.qgemm_host_band_schedule(int(extent), int(bands), 1 if shrink else 0, buf, n)
    return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(n)]


def gemm_host(a_host, b_host, c_host, scale_a=None, scale_b=None, b_kmajor: bool = False, device=None) -> None:
    """c_host[M,N] = cast(scale_a*scale_b*(a_host[M,K] x B)) with all three tensors in (pinned) host memory;
    B = b_host[K,N], or b_host[N,K] with ``b_kmajor``. ``scale_a`` / ``scale_b`` are Python floats or None.
    Enqueues on the current stream of ``device`` (default: the current device); synchronise that stream
    before reading ``c_host``."""
    for name, t in (("a_host", a_host), ("b_host", b_host), ("c_host", c_host)):
        if t.is_cuda or t.dim() != 2 or (t.stride(1) != 1 and t.shape[1] > 1):
            raise QgemmError(ERR_INVALID_ARG, f"{name} must be a 2-D host tensor with unit inner stride")
    M, K = a_host.shape
    N, Kb = (b_host.shape[0], b_host.shape[1]) if b_kmajor else (b_host.shape[1], b_host.shape[0])
    if Kb != K or tuple(c_host.shape) != (M, N) or a_host.dtype != b_host.dtype:
        raise QgemmError(ERR_INVALID_ARG, "shape or dtype mismatch")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    sa = C.byref(C.c_float(float(scale_a))) if scale_a is not None else None
    sb = C.byref(C.c_float(float(scale_b))) if scale_b is not None else None
    with torch.cuda.device(dev):
        rc = lib().qgemm_gemm_host(
            _dtype_code(a_host), _dtype_code(c_host), B_K_MAJOR if b_kmajor else B_ROW_MAJOR,
            a_host.data_ptr(), max(a_host.stride(0), K), b_host.data_ptr(), max(b_host.stride(0), b_host.shape[1]),
            sa, sb, c_host.data_ptr(), max(c_host.stride(0), N), M, N, K,
            torch.cuda.current_stream(dev).cuda_stream)
    _check(rc, "qgemm_gemm_host")


class HostGemm:
    """One problem shape on host operands. Kept as a class so that callers can query the traffic and the
    launch count of a call; the device buffers live inside the library."""

    def __init__(self, M: int, N: int, K: int, in_dtype, out_dtype, b_kmajor: bool, device, bands: int = 8):
        self.M, self.N, self.K = M, N, K
        self.b_kmajor = b_kmajor
        self.device = torch.device(device)
        self.in_dtype, self.out_dtype = in_dtype, out_dtype
        es = torch.empty((), dtype=in_dtype).element_size()
        osz = torch.empty((), dtype=out_dtype).element_size()
        self.h2d_bytes = (M * K + N * K) * es
        self.d2h_bytes = M * N * osz
        # one GEMM per arriving band except the very first (nothing to multiply it with yet)
        self.kernel_launches_per_call = max(1, len(band_schedule(M, bands)) + len(band_schedule(N, bands, False)) - 1)

    def __call__(self, a_host, b_host, c_host, scale_a=None, scale_b=None) -> None:
        """Enqueue one C = A x B with pinned host tensors on the current stream's dependency chain
        (synchronise the current stream to wait for c_host). Scales: floats, 1-element tensors or None."""
        def as_float(s):
            if s is None:
                return None
            return float(s.item()) if hasattr(s, "item") else float(s)
        gemm_host(a_host, b_host, c_host, as_float(scale_a), as_float(scale_b), self.b_kmajor, self.device)
