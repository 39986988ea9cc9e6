"""qgemm_b200 -- Python host side of the B200 (sm_100a) quantized-GEMM library.

The product is ``libqgemm.so`` (hand-written CUDA behind the C-ABI of ``include/qgemm.h``). This
package loads it with ctypes and mirrors the torch-level entry points the reference sketches
(``bf16_mm`` / ``int8_mm`` / ``fp8_mm`` taking ``(a, b, as, bs, c)``,
src/gemm/sm80_gemm_kernel.cu:4-22 and src/mix_gemm/hip_mix_gemm_kernel.cpp:508-516). PyTorch is
used only for device memory and streams; there is no CPU or eager fallback -- if the shared
library is missing, importing :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
#: the library to load; QGEMM_LIBRARY names another build of it (e.g. the diagnostic one of ``build.py --stamps``)
LIB_PATH = os.environ.get("QGEMM_LIBRARY") or os.path.join(HERE, "libqgemm.so")

# qgemm_status_t
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_WORKSPACE, ERR_DEVICE_TIMEOUT = range(7)
# qgemm_dtype_t
BF16, FP16, INT8, FP8_E4M3, FP32, INT32, INT4 = range(7)
# qgemm_b_layout_t
B_ROW_MAJOR, B_K_MAJOR = 0, 1

#: every symbol include/qgemm.h declares
C_ABI_SYMBOLS = (
    "qgemm_gemm", "qgemm_mix_gemm", "qgemm_gemm_ex", "qgemm_transpose", "qgemm_workspace_reserve",
    "qgemm_workspace_bytes", "qgemm_workspace_query", "qgemm_device_status", "qgemm_shutdown",
    "qgemm_status_string", "qgemm_version", "qgemm_mix_gemm_splitk_static",
    "qgemm_fp8_block_scaled_gemm", "qgemm_quantize", "qgemm_gemm_multi_dst", "qgemm_peer_export",
    "qgemm_peer_open", "qgemm_peer_close", "qgemm_gemm_host", "qgemm_plan_query", "qgemm_host_band_schedule",
    "qgemm_gemm_host_resident_a", "qgemm_plan_query_ex", "qgemm_peer_alloc", "qgemm_peer_free", "qgemm_reload_env", "qgemm_test_arm_skip_load",
)


class Tuning(C.Structure):
    """qgemm_tuning_t: zero fields mean "library heuristic"."""
    _fields_ = [("tile_n", C.c_int), ("split_k", C.c_int), ("group_m", C.c_int), ("max_ctas", C.c_int),
                ("cta_pair", C.c_int), ("relayout_b", C.c_int)]


class QgemmError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} (status {status})")


_lib = None


def lib() -> C.CDLL:
    """The loaded C-ABI library. Raises if it has not been built (python -m qgemm_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m qgemm_b200.build`; "
                              "there is no fallback path")
        L = C.CDLL(LIB_PATH)
        sz, vp, fp, i = C.c_size_t, C.c_void_p, C.c_void_p, C.c_int
        L.qgemm_gemm.argtypes = [i, i, i, vp, sz, vp, sz, vp, sz, sz, sz, sz, vp]
        L.qgemm_mix_gemm.argtypes = [i, i, i, vp, sz, vp, sz, fp, fp, vp, sz, sz, sz, sz, vp]
        L.qgemm_gemm_ex.argtypes = [i, i, i, vp, sz, vp, sz, fp, fp, vp, sz, sz, sz, sz, C.POINTER(Tuning), vp]
        L.qgemm_transpose.argtypes = [vp, vp, sz, sz, sz, sz, sz, vp]
        L.qgemm_workspace_reserve.argtypes = [sz]
        L.qgemm_workspace_bytes.restype = sz
        L.qgemm_workspace_query.argtypes = [i, i, sz, sz, sz, C.POINTER(Tuning)]
        L.qgemm_workspace_query.restype = sz
        L.qgemm_device_status.argtypes = [C.POINTER(C.c_int)]
        L.qgemm_status_string.argtypes = [i]
        L.qgemm_status_string.restype = C.c_char_p
        L.qgemm_mix_gemm_splitk_static.argtypes = [i, i, vp, sz, vp, sz, fp, fp, vp, sz, sz, sz, sz, i, vp]
        L.qgemm_mix_gemm_splitk_static.restype = i
        L.qgemm_fp8_block_scaled_gemm.argtypes = [i, i, i, vp, sz, vp, sz, fp, fp, vp, sz, sz, sz, sz, vp]
        L.qgemm_fp8_block_scaled_gemm.restype = i
        L.qgemm_quantize.argtypes = [i, i, vp, sz, vp, sz, fp, fp, sz, sz, vp]
        L.qgemm_quantize.restype = i
        L.qgemm_gemm_multi_dst.argtypes = [i, i, i, vp, sz, vp, sz, fp, fp, C.POINTER(C.c_void_p), i, sz, sz, sz, sz, vp]
        L.qgemm_gemm_multi_dst.restype = i
        L.qgemm_gemm_host.argtypes = [i, i, i, vp, sz, vp, sz, C.POINTER(C.c_float), C.POINTER(C.c_float), vp, sz, sz,
                                      sz, sz, vp]
        L.qgemm_gemm_host.restype = i
        L.qgemm_plan_query.argtypes = [i, i, i, sz, sz, sz, C.POINTER(Tuning), C.POINTER(C.c_int)]
        L.qgemm_plan_query.restype = i
        L.qgemm_plan_query_ex.argtypes = [i, i, i, sz, sz, sz, C.POINTER(Tuning), C.POINTER(C.c_int), i]
        L.qgemm_plan_query_ex.restype = i
        L.qgemm_gemm_host_resident_a.argtypes = L.qgemm_gemm_host.argtypes
        L.qgemm_gemm_host_resident_a.restype = i
        L.qgemm_host_band_schedule.argtypes = [sz, i, i, C.POINTER(sz), i]
        L.qgemm_host_band_schedule.restype = i
        L.qgemm_reload_env.restype = i
        L.qgemm_test_arm_skip_load.argtypes = [i]
        L.qgemm_test_arm_skip_load.restype = i
        L.qgemm_peer_alloc.argtypes = [sz, C.POINTER(C.c_void_p)]
        L.qgemm_peer_alloc.restype = i
        L.qgemm_peer_free.argtypes = [vp]
        L.qgemm_peer_free.restype = i
        L.qgemm_peer_export.argtypes = [vp, vp, C.POINTER(sz)]
        L.qgemm_peer_export.restype = i
        L.qgemm_peer_open.argtypes = [vp, C.POINTER(C.c_void_p)]
        L.qgemm_peer_open.restype = i
        L.qgemm_peer_close.argtypes = [vp]
        L.qgemm_peer_close.restype = i
        for name in ("qgemm_gemm", "qgemm_mix_gemm", "qgemm_gemm_ex", "qgemm_transpose", "qgemm_workspace_reserve",
                     "qgemm_device_status", "qgemm_shutdown", "qgemm_version"):
            getattr(L, name).restype = i
        _lib = L
    return _lib


def status_string(status: int) -> str:
    return lib().qgemm_status_string(int(status)).decode()


def _check(status: int, what: str) -> None:
    if status != OK:
        raise QgemmError(status, what)


# ----------------------------------------------------------------------------- torch-level API
def _torch():
    import torch
    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    table = {torch.bfloat16: BF16, torch.float16: FP16, torch.int8: INT8, torch.float32: FP32, torch.int32: INT32}
    if hasattr(torch, "float8_e4m3fn"):
        table[torch.float8_e4m3fn] = FP8_E4M3
    if t.dtype not in table:
        raise QgemmError(ERR_UNSUPPORTED, f"dtype {t.dtype}")
    return table[t.dtype]


def _require_cuda_2d(name, t):
    if not t.is_cuda:
        raise QgemmError(ERR_INVALID_ARG, f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dim() != 2 or (t.stride(1) != 1 and t.shape[1] > 1):
        raise QgemmError(ERR_INVALID_ARG, f"{name} must be 2-D with unit inner stride")


def _stream_ptr(t) -> int:
    return _torch().cuda.current_stream(t.device).cuda_stream


def _gemm(a, b, scale_a, scale_b, c, b_kmajor: bool, tuning: Tuning | None, mixed: bool) -> None:
    torch = _torch()
    for name, t in (("a", a), ("b", b), ("c", c)):
        _require_cuda_2d(name, t)
    if a.dtype != b.dtype:
        raise QgemmError(ERR_INVALID_ARG, "a and b must have the same dtype")
    M, K = a.shape
    if b_kmajor:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    if Kb != K or tuple(c.shape) != (M, N):
        raise QgemmError(ERR_INVALID_ARG, f"shape mismatch a{tuple(a.shape)} b{tuple(b.shape)} c{tuple(c.shape)}")
    for name, s in (("scale_a", scale_a), ("scale_b", scale_b)):
        if s is not None and (not s.is_cuda or s.dtype != torch.float32 or s.numel() != 1):
            raise QgemmError(ERR_INVALID_ARG, f"{name} must be a 1-element float32 CUDA tensor")
    sa = scale_a.data_ptr() if scale_a is not None else None
    sb = scale_b.data_ptr() if scale_b is not None else None
    with torch.cuda.device(a.device):
        rc = lib().qgemm_gemm_ex(
            _dtype_code(a), _dtype_code(c), B_K_MAJOR if b_kmajor else B_ROW_MAJOR,
            a.data_ptr(), max(a.stride(0), K), b.data_ptr(), max(b.stride(0), b.shape[1]),
            sa, sb, c.data_ptr(), max(c.stride(0), N), M, N, K,
            C.byref(tuning) if tuning is not None else None, _stream_ptr(a))
    _check(rc, "qgemm_gemm_ex" if not mixed else "qgemm_mix_gemm")


def gemm(a, b, c, b_kmajor: bool = False, tuning: Tuning | None = None) -> None:
    """c[M,N] = a[M,K] x B, B = b[K,N] (row-major) or, with ``b_kmajor``, b[N,K].

    bf16/fp16 inputs give fp32/bf16/fp16 output with fp32 accumulation; int8 inputs give the exact
    int32 accumulator. Mirrors GEMM_kernel_vN<typeIn,typeOut> of the reference's include/gemm.h:25-66.
    """
    _gemm(a, b, None, None, c, b_kmajor, tuning, mixed=False)


def mix_gemm(a, b, scale_a, scale_b, c, b_kmajor: bool = True, tuning: Tuning | None = None) -> None:
    """c = cast(scale_a * scale_b * (a x B)) for int8 (int32 accumulate) or fp8-e4m3 (fp32 accumulate)."""
    _gemm(a, b, scale_a, scale_b, c, b_kmajor, tuning, mixed=True)


def bf16_mm(a, b, a_scale, b_scale, c) -> None:
    """(a, b, as, bs, c) with a [m,k], b [n,k] as the reference's torch entry points take them
    (n = b.size(0), src/gemm/sm80_gemm_kernel.cu:4-12). Scales may be None."""
    _gemm(a, b, a_scale, b_scale, c, True, None, mixed=True)


def int8_mm(a, b, a_scale, b_scale, c) -> None:
    """int8 a [m,k], b [n,k], per-matrix float32 scales -> c [m,n] (src/gemm/sm80_gemm_kernel.cu:14-22)."""
    _gemm(a, b, a_scale, b_scale, c, True, None, mixed=True)


def fp8_mm(a, b, a_scale, b_scale, c) -> None:
    """fp8-e4m3 a [m,k], b [n,k], per-matrix float32 scales -> c [m,n]
    (src/mix_gemm/hip_mix_gemm_kernel.cpp:508-516; per-matrix instead of block scales)."""
    _gemm(a, b, a_scale, b_scale, c, True, None, mixed=True)


A_ROW_MAJOR, A_COL_MAJOR = 0, 1


def int4_mm(a_packed, b_packed, a_scale, b_scale, c, tuning: Tuning | None = None) -> None:
    """Int4 mixed GEMM (the "Int4" precision of the reference's roadmap, develop.md:9-12): ``a_packed`` [m, k/2] and
    ``b_packed`` [n, k/2] are uint8 / int8 tensors holding two signed 4-bit values per byte (element 2i in the low
    nibble), K-major. ``c`` [m, n]: int32 (exact sums, both scales None) or bf16 / fp16 / fp32 =
    cast(a_scale * b_scale * sum). The operands are widened to int8 on the device and multiplied by the int8 kernel."""
    torch = _torch()
    for name, t in (("a_packed", a_packed), ("b_packed", b_packed), ("c", c)):
        _require_cuda_2d(name, t)
    if a_packed.element_size() != 1 or b_packed.element_size() != 1:
        raise QgemmError(ERR_INVALID_ARG, "packed int4 operands are 1-byte tensors (two values per byte)")
    M, Kh = a_packed.shape
    N = b_packed.shape[0]
    if b_packed.shape[1] != Kh or tuple(c.shape) != (M, N):
        raise QgemmError(ERR_INVALID_ARG, "shape mismatch")
    sa = a_scale.data_ptr() if a_scale is not None else None
    sb = b_scale.data_ptr() if b_scale is not None else None
    with torch.cuda.device(a_packed.device):
        rc = lib().qgemm_gemm_ex(INT4, _dtype_code(c), B_K_MAJOR, a_packed.data_ptr(), 2 * max(a_packed.stride(0), Kh),
                                 b_packed.data_ptr(), 2 * max(b_packed.stride(0), Kh), sa, sb, c.data_ptr(),
                                 max(c.stride(0), N), M, N, 2 * Kh, C.byref(tuning) if tuning is not None else None,
                                 _stream_ptr(a_packed))
    _check(rc, "qgemm_gemm_ex (int4)")


def quantize_int4(x, out=None):
    """Per-matrix int4 quantisation of a float32 / bfloat16 CUDA matrix with an even number of columns. Returns
    ``(packed, scale)``: ``packed`` uint8 [rows, cols/2] (two values per byte, low nibble first), ``scale`` =
    amax / 7 as a 1-element float32 CUDA tensor."""
    torch = _torch()
    _require_cuda_2d("x", x)
    rows, cols = x.shape
    if cols % 2:
        raise QgemmError(ERR_INVALID_ARG, "int4 packs two values per byte: the number of columns must be even")
    if out is None:
        out = torch.empty((rows, cols // 2), dtype=torch.uint8, device=x.device)
    _require_cuda_2d("out", out)
    if tuple(out.shape) != (rows, cols // 2) or out.element_size() != 1:
        raise QgemmError(ERR_INVALID_ARG, "out must be a 1-byte tensor of shape [rows, cols/2]")
    sc = torch.empty(2, dtype=torch.float32, device=x.device)  # [scale, amax]
    with torch.cuda.device(x.device):
        rc = lib().qgemm_quantize(_dtype_code(x), INT4, x.data_ptr(), max(x.stride(0), cols), out.data_ptr(),
                                  2 * max(out.stride(0), cols // 2), sc.data_ptr(), sc.data_ptr() + 4, rows, cols,
                                  _stream_ptr(x))
    _check(rc, "qgemm_quantize (int4)")
    return out, sc[:1]


def quantize(x, out_dtype, out=None):
    """Per-matrix quantisation of a float32 / bfloat16 CUDA matrix to ``torch.float8_e4m3fn`` or ``torch.int8``.
    Returns ``(q, scale)`` with ``scale`` a 1-element float32 CUDA tensor (amax/448 or amax/127) ready to be
    passed to :func:`mix_gemm`; nothing is synchronised or copied to the host."""
    torch = _torch()
    _require_cuda_2d("x", x)
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=out_dtype, device=x.device)
    _require_cuda_2d("out", out)
    if tuple(out.shape) != (rows, cols) or out.dtype != out_dtype:
        raise QgemmError(ERR_INVALID_ARG, "out must have the input's shape and the requested dtype")
    sc = torch.empty(2, dtype=torch.float32, device=x.device)  # [scale, amax]
    with torch.cuda.device(x.device):
        rc = lib().qgemm_quantize(_dtype_code(x), _dtype_code(out), x.data_ptr(), max(x.stride(0), cols),
                                  out.data_ptr(), max(out.stride(0), cols), sc.data_ptr(), sc.data_ptr() + 4, rows,
                                  cols, _stream_ptr(x))
    _check(rc, "qgemm_quantize")
    return out, sc[:1]


def fp8_block_mm(a, b, a_scale, b_scale, c, reference_layout: bool = True) -> None:
    """Block-scaled FP8 GEMM, fp8_mm(a, b, as, bs, c) of src/mix_gemm/hip_mix_gemm_kernel.cpp:425-439,508-516.

    With ``reference_layout`` the operands are laid out as the reference takes them: ``a`` is the
    [m,k] matrix stored column-major, i.e. a contiguous tensor of shape [k, m]; ``b`` is [n,k]
    column-major, i.e. a contiguous [k, n]; otherwise ``a`` is [m,k] and ``b`` is [n,k], both row-major
    (K-major). ``a_scale`` [ceil(k/128), m] and ``b_scale`` [ceil(k/128), ceil(n/128)] are float32 (the
    reference's "[m, k/128] col-major" and "[k/128, n/128] row-major"). ``c`` [m,n] bf16/fp16/fp32."""
    torch = _torch()
    for name, t in (("a", a), ("b", b), ("c", c), ("a_scale", a_scale), ("b_scale", b_scale)):
        _require_cuda_2d(name, t)
    M, N = c.shape
    if reference_layout:
        K = a.shape[0]
        ok = tuple(a.shape) == (K, M) and tuple(b.shape) == (K, N)
        a_layout, b_layout = A_COL_MAJOR, B_ROW_MAJOR
    else:
        K = a.shape[1]
        ok = tuple(a.shape) == (M, K) and tuple(b.shape) == (N, K)
        a_layout, b_layout = A_ROW_MAJOR, B_K_MAJOR
    kbs, nbs = -(-K // 128), -(-N // 128)
    ok = ok and tuple(a_scale.shape) == (kbs, M) and tuple(b_scale.shape) == (kbs, nbs)
    ok = ok and a_scale.dtype == torch.float32 and b_scale.dtype == torch.float32
    ok = ok and a_scale.is_contiguous() and b_scale.is_contiguous()
    if not ok or _dtype_code(a) != FP8_E4M3 or _dtype_code(b) != FP8_E4M3:
        raise QgemmError(ERR_INVALID_ARG, "fp8_block_mm: shape, dtype or layout mismatch")
    with torch.cuda.device(a.device):
        rc = lib().qgemm_fp8_block_scaled_gemm(
            _dtype_code(c), a_layout, b_layout, a.data_ptr(), max(a.stride(0), a.shape[1]), b.data_ptr(),
            max(b.stride(0), b.shape[1]), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(), max(c.stride(0), N),
            M, N, K, _stream_ptr(a))
    _check(rc, "qgemm_fp8_block_scaled_gemm")


MAX_DSTS = 8  # QGEMM_MAX_DSTS
PEER_HANDLE_BYTES = 64  # QGEMM_PEER_HANDLE_BYTES


def gemm_multi_dst(a, b, scale_a, scale_b, dst_ptrs, ldc: int, out_dtype, n_cols: int, b_kmajor: bool = True) -> None:
    """One GEMM whose [M, n_cols] result is stored to every address of ``dst_ptrs`` (device addresses, this
    GPU's or mapped from other GPUs with :func:`peer_open`), all with leading dimension ``ldc`` elements of
    ``out_dtype``. The column-sharded configuration uses it to leave the gathered C on every GPU from the
    GEMM's own epilogue. Enqueues on the current stream of ``a``'s device; the caller synchronises and lets
    the ranks meet before anybody reads."""
    torch = _torch()
    _require_cuda_2d("a", a)
    _require_cuda_2d("b", b)
    M, K = a.shape
    N, Kb = (b.shape[0], b.shape[1]) if b_kmajor else (b.shape[1], b.shape[0])
    if Kb != K or N != n_cols or a.dtype != b.dtype:
        raise QgemmError(ERR_INVALID_ARG, "shape or dtype mismatch")
    if not (1 <= len(dst_ptrs) <= MAX_DSTS):
        raise QgemmError(ERR_INVALID_ARG, f"between 1 and {MAX_DSTS} destinations")
    codes = {torch.bfloat16: BF16, torch.float16: FP16, torch.float32: FP32, torch.int32: INT32}
    if out_dtype not in codes:
        raise QgemmError(ERR_UNSUPPORTED, f"output dtype {out_dtype}")
    arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    sa = scale_a.data_ptr() if scale_a is not None else None
    sb = scale_b.data_ptr() if scale_b is not None else None
    with torch.cuda.device(a.device):
        rc = lib().qgemm_gemm_multi_dst(
            _dtype_code(a), codes[out_dtype], B_K_MAJOR if b_kmajor else B_ROW_MAJOR, a.data_ptr(),
            max(a.stride(0), K), b.data_ptr(), max(b.stride(0), b.shape[1]), sa, sb, arr, len(dst_ptrs), int(ldc),
            M, N, K, _stream_ptr(a))
    _check(rc, "qgemm_gemm_multi_dst")


class _DeviceBlock:
    """A cudaMalloc'ed block of its own, seen by torch through the CUDA array interface (no copy); freed when the
    last tensor that views it is gone and :meth:`free` has been called, or at interpreter exit."""

    def __init__(self, nbytes: int, device):
        torch = _torch()
        self.device = torch.device(device)
        ptr = C.c_void_p(0)
        with torch.cuda.device(self.device):
            _check(lib().qgemm_peer_alloc(int(nbytes), C.byref(ptr)), "qgemm_peer_alloc")
        self.ptr, self.nbytes = int(ptr.value), int(nbytes)
        self.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1", "data": (self.ptr, False),
                                         "version": 2}

    def free(self) -> None:
        if self.ptr:
            with _torch().cuda.device(self.device):
                _check(lib().qgemm_peer_free(C.c_void_p(self.ptr)), "qgemm_peer_free")
            self.ptr = 0


def peer_tensor(shape, dtype, device):
    """(tensor, block): a tensor of ``shape`` / ``dtype`` in a device allocation of its own, so that exporting it with
    :func:`peer_export` exposes nothing else of this process. Call ``block.free()`` when every peer has unmapped it
    and the tensor is no longer used."""
    torch = _torch()
    n = 1
    for d in shape:
        n *= int(d)
    block = _DeviceBlock(max(1, n * torch.empty((), dtype=dtype).element_size()), device)
    flat = torch.as_tensor(block, device=torch.device(device))
    return flat.view(dtype).view(*shape), block


def peer_export(t):
    """(handle bytes, byte offset) of a CUDA tensor's storage for another process of this box to map."""
    torch = _torch()
    handle = C.create_string_buffer(PEER_HANDLE_BYTES)
    offset = C.c_size_t(0)
    with torch.cuda.device(t.device):
        _check(lib().qgemm_peer_export(t.data_ptr(), handle, C.byref(offset)), "qgemm_peer_export")
    return handle.raw, int(offset.value)


def peer_open(handle: bytes, device) -> int:
    """Maps an exported allocation into this process on ``device``; returns its base address."""
    torch = _torch()
    base = C.c_void_p(0)
    buf = C.create_string_buffer(bytes(handle), PEER_HANDLE_BYTES)
    with torch.cuda.device(device):
        _check(lib().qgemm_peer_open(buf, C.byref(base)), "qgemm_peer_open")
    return int(base.value)


def peer_close(base: int, device) -> None:
    with _torch().cuda.device(device):
        _check(lib().qgemm_peer_close(C.c_void_p(base)), "qgemm_peer_close")


STATIC_SCRATCH_BYTES = 32 << 20  # QGEMM_STATIC_SCRATCH_BYTES


def mix_gemm_splitk_static(a, b, scale_a, scale_b, c, split_k: int) -> None:
    """Split-K GEMM through the entry point that never allocates (for callers that cannot call
    cudaMalloc where they need the product: fixed-budget embedders, loops that must not risk a
    device-wide synchronisation, processes whose GPU memory is already owned by another allocator).
    a [M,K], b [N,K] K-major; partial sums live in a fixed ``STATIC_SCRATCH_BYTES`` array inside the
    library, so ``split_k * M * round_up(N, 4) * 4`` must fit in it and calls that overlap on the GPU
    must be serialised by the caller. Bit-identical to ``mix_gemm(..., tuning=Tuning(128, split_k, 0, 0))``."""
    torch = _torch()
    for name, t in (("a", a), ("b", b), ("c", c)):
        _require_cuda_2d(name, t)
    M, K = a.shape
    N = b.shape[0]
    if b.shape[1] != K or tuple(c.shape) != (M, N) or a.dtype != b.dtype:
        raise QgemmError(ERR_INVALID_ARG, "shape or dtype mismatch")
    sa = scale_a.data_ptr() if scale_a is not None else None
    sb = scale_b.data_ptr() if scale_b is not None else None
    with torch.cuda.device(a.device):
        rc = lib().qgemm_mix_gemm_splitk_static(
            _dtype_code(a), _dtype_code(c), a.data_ptr(), max(a.stride(0), K), b.data_ptr(), max(b.stride(0), K),
            sa, sb, c.data_ptr(), max(c.stride(0), N), M, N, K, int(split_k), _stream_ptr(a))
    _check(rc, "qgemm_mix_gemm_splitk_static")


def transpose(x, out=None):
    """out[c, r] = x[r, c] for 1- or 2-byte element tensors (matrix_transpose<T>,
    src/include/matrix_transpose.h:3-4)."""
    torch = _torch()
    _require_cuda_2d("x", x)
    rows, cols = x.shape
    if out is None:
        out = torch.empty((cols, rows), dtype=x.dtype, device=x.device)
    _require_cuda_2d("out", out)
    if tuple(out.shape) != (cols, rows) or out.dtype != x.dtype:
        raise QgemmError(ERR_INVALID_ARG, "out must be [cols, rows] of the same dtype")
    with torch.cuda.device(x.device):
        rc = lib().qgemm_transpose(x.data_ptr(), out.data_ptr(), rows, cols, max(x.stride(0), cols),
                                   max(out.stride(0), rows),
                                   x.element_size(), _stream_ptr(x))
    _check(rc, "qgemm_transpose")
    return out


def workspace_reserve(nbytes: int) -> None:
    _check(lib().qgemm_workspace_reserve(int(nbytes)), "qgemm_workspace_reserve")


def workspace_query(in_dtype: int, b_layout: int, M: int, N: int, K: int, tuning: Tuning | None = None) -> int:
    return int(lib().qgemm_workspace_query(in_dtype, b_layout, M, N, K, C.byref(tuning) if tuning else None))


def plan_query(in_dtype: int, out_dtype: int, b_layout: int, M: int, N: int, K: int, tuning: Tuning | None = None):
    """The kernel configuration the library would use for this shape (qgemm_plan_query_ex): tile_m, tile_n,
    ctas_per_tile, split_k, tail_tiles, tail_slices, balanced_tiles (tile columns of the balanced tiling, 0 = equal
    tiles), min_tile_n, a_rows_per_stage, ctas, cluster_slices (CTAs per cluster when the K slices are added up inside
    one launch, else 0), k_blocks_per_load."""
    n = 12
    out = (C.c_int * n)()
    _check(lib().qgemm_plan_query_ex(in_dtype, out_dtype, b_layout, M, N, K, C.byref(tuning) if tuning else None, out,
                                     n), "qgemm_plan_query_ex")
    keys = ("tile_m", "tile_n", "ctas_per_tile", "split_k", "tail_tiles", "tail_slices", "balanced_tiles",
            "min_tile_n", "a_rows_per_stage", "ctas", "cluster_slices", "k_blocks_per_load")
    return dict(zip(keys, list(out)))


def device_status():
    """Synchronise and return (status, [code, cta, role, position])."""
    buf = (C.c_int * 4)()
    rc = lib().qgemm_device_status(buf)
    return rc, list(buf)


def shutdown() -> None:
    _check(lib().qgemm_shutdown(), "qgemm_shutdown")
