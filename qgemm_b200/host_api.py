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


def gemm_host_resident_a(a_dev, b_host, c_host, scale_a=None, scale_b=None, b_kmajor: bool = False) -> None:
    """As :func:`gemm_host` with A already on the device (``qgemm_gemm_host_resident_a``): only B goes up, band by
    band, each followed by the GEMM and the download of the column strip of C it completes. Enqueues after the
    current stream of ``a_dev``'s device."""
    if not a_dev.is_cuda or a_dev.dim() != 2 or a_dev.stride(1) != 1:
        raise QgemmError(ERR_INVALID_ARG, "a_dev must be a 2-D CUDA tensor with unit inner stride")
    for name, t in (("b_host", b_host), ("c_host", c_host)):
        if t.is_cuda or t.dim() != 2 or (t.stride(1) != 1 and t.shape[1] > 1):
            raise QgemmError(ERR_INVALID_ARG, f"{name} must be a 2-D host tensor with unit inner stride")
    M, K = a_dev.shape
    N, Kb = (b_host.shape[0], b_host.shape[1]) if b_kmajor else (b_host.shape[1], b_host.shape[0])
    if Kb != K or tuple(c_host.shape) != (M, N) or a_dev.dtype != b_host.dtype:
        raise QgemmError(ERR_INVALID_ARG, "shape or dtype mismatch")
    sa = C.byref(C.c_float(float(scale_a))) if scale_a is not None else None
    sb = C.byref(C.c_float(float(scale_b))) if scale_b is not None else None
    with torch.cuda.device(a_dev.device):
        rc = lib().qgemm_gemm_host_resident_a(
            _dtype_code(a_dev), _dtype_code(c_host), B_K_MAJOR if b_kmajor else B_ROW_MAJOR,
            a_dev.data_ptr(), max(a_dev.stride(0), K), b_host.data_ptr(), max(b_host.stride(0), b_host.shape[1]),
            sa, sb, c_host.data_ptr(), max(c_host.stride(0), N), M, N, K,
            torch.cuda.current_stream(a_dev.device).cuda_stream)
    _check(rc, "qgemm_gemm_host_resident_a")


class HostGemm:
    """One problem shape on host operands. Kept as a class so that callers can query the traffic and the
    launch count of a call; the device buffers of B and C live inside the library.

    ``shared_a_group``: a ``torch.distributed`` group whose ranks all multiply the SAME A by their own B (the
    column-sharded product). Then every call is collective: rank r uploads only rows [r*M/W, (r+1)*M/W) of A, the
    ranks all-gather the row blocks over NVLink into each one's device copy of A, and B follows band by band
    (``qgemm_gemm_host_resident_a``). A crosses PCIe once per box instead of once per GPU."""

    def __init__(self, M: int, N: int, K: int, in_dtype, out_dtype, b_kmajor: bool, device, bands: int = 8,
                 shared_a_group=None):
        self.M, self.N, self.K = M, N, K
        self.b_kmajor = b_kmajor
        self.device = torch.device(device)
        self.in_dtype, self.out_dtype = in_dtype, out_dtype
        es = torch.empty((), dtype=in_dtype).element_size()
        osz = torch.empty((), dtype=out_dtype).element_size()
        self.group = shared_a_group
        self.world = 1
        self.nvlink_bytes = 0
        self.a_upload = "whole A by this rank"
        self._a_dev = None
        if shared_a_group is not None:
            import torch.distributed as dist
            self.world = dist.get_world_size(shared_a_group)
            self.rank = dist.get_rank(shared_a_group)
        if self.world > 1 and M % self.world == 0:
            self._a_dev = torch.empty((M, K), dtype=in_dtype, device=self.device)
            self.h2d_bytes = (M // self.world * K + N * K) * es
            self.nvlink_bytes = (M - M // self.world) * K * es
            self.a_upload = (f"rows [r*M/{self.world}, (r+1)*M/{self.world}) by rank r, all-gathered over NVLink "
                             "(NCCL) into every rank's device copy")
            self.kernel_launches_per_call = len(band_schedule(N, bands, False))
        else:
            self.world = 1
            self.h2d_bytes = (M * K + N * K) * es
            # one GEMM per arriving band except the very first (nothing to multiply it with yet)
            self.kernel_launches_per_call = max(1, len(band_schedule(M, bands)) + len(band_schedule(N, bands, False)) - 1)
        self.d2h_bytes = M * N * osz

    def __call__(self, a_host, b_host, c_host, scale_a=None, scale_b=None) -> None:
        """Enqueue one C = A x B with pinned host tensors on the current stream's dependency chain
        (synchronise the current stream to wait for c_host). Scales: floats, 1-element tensors or None."""
        def as_float(s):
            if s is None:
                return None
            return float(s.item()) if hasattr(s, "item") else float(s)
        if self._a_dev is None:
            gemm_host(a_host, b_host, c_host, as_float(scale_a), as_float(scale_b), self.b_kmajor, self.device)
            return
        import torch.distributed as dist
        rows = self.M // self.world
        mine = self._a_dev[self.rank * rows:(self.rank + 1) * rows]
        with torch.cuda.device(self.device):
            mine.copy_(a_host[self.rank * rows:(self.rank + 1) * rows], non_blocking=True)
            # in place: every rank's block already sits where the gathered matrix wants it
            dist.all_gather_into_tensor(self._a_dev, mine, group=self.group)
        gemm_host_resident_a(self._a_dev, b_host, c_host, as_float(scale_a), as_float(scale_b), self.b_kmajor)

    def copy_only(self, a_host, b_host, c_host, ctx, steps: int = 5) -> dict:
        """The ceiling the host side sets for a step: the step's own host-to-device and device-to-host bytes copied
        concurrently on two streams with no GEMM in between, every rank at once; aggregate GB/s over all ranks,
        timed on the device, max over ranks."""
        dev = self.device
        rows = self.M // self.world
        a_src = a_host[:rows] if self._a_dev is not None else a_host
        a_d = torch.empty_like(a_src, device=dev)
        b_d = torch.empty_like(b_host, device=dev)
        c_d = torch.empty_like(c_host, device=dev)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def step():
            cur = torch.cuda.current_stream(dev)
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            with torch.cuda.stream(s_in):
                a_d.copy_(a_src, non_blocking=True)
                b_d.copy_(b_host, non_blocking=True)
            with torch.cuda.stream(s_out):
                c_host.copy_(c_d, non_blocking=True)
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)

        for _ in range(2):
            step()
        ms = ctx.max_over_ranks(ctx.timed(step, steps, False)[0]) / steps
        total = (self.h2d_bytes + self.d2h_bytes) * ctx.world
        return {"ms_per_step": ms, "aggregate_gbs": total / (ms * 1e-3) / 1e9,
                "h2d_gbs_per_rank": self.h2d_bytes / (ms * 1e-3) / 1e9,
                "d2h_gbs_per_rank": self.d2h_bytes / (ms * 1e-3) / 1e9,
                "note": "pinned host buffers, uploads and download on separate streams, no kernels"}
