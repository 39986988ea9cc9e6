"""ctypes/numpy front-end of the CPU oracle (``oracle/qgemm_oracle.c``).

TEST INFRASTRUCTURE ONLY: this module is the checker the CUDA kernels are compared with. The
library itself never imports it; only the tests, the smoke check and the CPU-baseline leg of the
benchmark do. Parity status is stated in the header of ``qgemm_oracle.c``.

All array arguments are numpy arrays; 16-bit and 8-bit floating formats travel as their raw bit
patterns (``uint16`` / ``uint8``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libqgemm_oracle.so")
_lib = None

OUT_F32, OUT_BF16, OUT_F16 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the C oracle with ``make`` if the shared object is missing or stale."""
    src = os.path.join(_HERE, "qgemm_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_quantize_e4m3.restype = C.c_float
        _lib.oracle_quantize_int8.restype = C.c_float
        _lib.oracle_quantize_int4.restype = C.c_float
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _sz(x):
    return C.c_size_t(int(x))


def set_threads(n: int) -> None:
    lib().oracle_set_threads(C.c_int(int(n)))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


# ---------------------------------------------------------------- conversions
def round_bf16(x: np.ndarray):
    """fp32 -> (bf16 bit patterns, the rounded values as fp32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = np.empty(x.shape, np.uint16)
    val = np.empty(x.shape, np.float32)
    lib().oracle_round_bf16(_p(x), _p(bits), _p(val), _sz(x.size))
    return bits, val


def round_f16(x: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = np.empty(x.shape, np.uint16)
    val = np.empty(x.shape, np.float32)
    lib().oracle_round_f16(_p(x), _p(bits), _p(val), _sz(x.size))
    return bits, val


def quantize_e4m3(x: np.ndarray):
    """Per-matrix FP8 quantisation: returns (e4m3 bit patterns, decoded values as fp32, scale)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = np.empty(x.shape, np.uint8)
    val = np.empty(x.shape, np.float32)
    scale = lib().oracle_quantize_e4m3(_p(x), _p(bits), _p(val), _sz(x.size))
    return bits, val, float(scale)


def quantize_int8(x: np.ndarray):
    """Per-matrix int8 quantisation: returns (int8 values, scale = amax/127)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    q = np.empty(x.shape, np.int8)
    scale = lib().oracle_quantize_int8(_p(x), _p(q), _sz(x.size))
    return q, float(scale)


def unpack_int4(packed: np.ndarray) -> np.ndarray:
    """Packed signed 4-bit [rows, cols/2] (two per byte, low nibble first) -> int8 [rows, cols]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.int8)
    lib().oracle_unpack_int4(_p(packed), _p(out), _sz(out.size))
    return out


def quantize_int4(x: np.ndarray):
    """Per-matrix int4 quantisation (scale = amax/7): returns (packed uint8 [rows, cols/2], scale)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % 2 == 0
    q = np.empty(x.shape[:-1] + (x.shape[-1] // 2,), np.uint8)
    scale = lib().oracle_quantize_int4(_p(x), _p(q), _sz(x.size))
    return q, float(scale)


def gemm_i4(A_packed: np.ndarray, Bt_packed: np.ndarray) -> np.ndarray:
    """Exact int32 product of packed int4 A [M, K/2] and K-major B [N, K/2]."""
    return gemm_i8(unpack_int4(A_packed), unpack_int4(Bt_packed), True)


def e4m3_decode(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint8)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_e4m3_decode(_p(bits), _p(out), _sz(bits.size))
    return out


def bf16_decode(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_bf16_decode(_p(bits), _p(out), _sz(bits.size))
    return out


def f16_decode(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_f16_decode(_p(bits), _p(out), _sz(bits.size))
    return out


# ---------------------------------------------------------------- GEMM
def _dims(A, B, b_kmajor):
    M, K = A.shape
    if b_kmajor:
        N, Kb = B.shape
    else:
        Kb, N = B.shape
    assert K == Kb, (A.shape, B.shape, b_kmajor)
    return M, N, K


def gemm_f32(A: np.ndarray, B: np.ndarray, b_kmajor: bool = False) -> np.ndarray:
    """C = A x B with sequential-k fp32 accumulation. B is [K,N], or [N,K] when ``b_kmajor``."""
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, N, K = _dims(A, B, b_kmajor)
    Cm = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32(_p(A), _sz(A.shape[1]), _p(B), _sz(B.shape[1]), C.c_int(int(b_kmajor)),
                          _p(Cm), _sz(N), _sz(M), _sz(N), _sz(K))
    return Cm


def gemm_f64(A: np.ndarray, B: np.ndarray, b_kmajor: bool = False) -> np.ndarray:
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, N, K = _dims(A, B, b_kmajor)
    Cm = np.empty((M, N), np.float64)
    lib().oracle_gemm_f64(_p(A), _sz(A.shape[1]), _p(B), _sz(B.shape[1]), C.c_int(int(b_kmajor)),
                          _p(Cm), _sz(N), _sz(M), _sz(N), _sz(K))
    return Cm


def gemm_i8(A: np.ndarray, B: np.ndarray, b_kmajor: bool = False) -> np.ndarray:
    A = np.ascontiguousarray(A, np.int8)
    B = np.ascontiguousarray(B, np.int8)
    M, N, K = _dims(A, B, b_kmajor)
    Cm = np.empty((M, N), np.int32)
    lib().oracle_gemm_i8(_p(A), _sz(A.shape[1]), _p(B), _sz(B.shape[1]), C.c_int(int(b_kmajor)),
                         _p(Cm), _sz(N), _sz(M), _sz(N), _sz(K))
    return Cm


def gemm_i8_rows(A: np.ndarray, Bt: np.ndarray, m0: int, m1: int) -> np.ndarray:
    """Rows [m0, m1) of A x Bt^T for K-major Bt [N,K]; exact int32."""
    A = np.ascontiguousarray(A, np.int8)
    Bt = np.ascontiguousarray(Bt, np.int8)
    N, K = Bt.shape
    assert A.shape[1] == K
    Cm = np.empty((m1 - m0, N), np.int32)
    lib().oracle_gemm_i8_rows(_p(A), _sz(K), _p(Bt), _sz(K), _p(Cm), _sz(N), _sz(m0), _sz(m1), _sz(N), _sz(K))
    return Cm


def gemm_f32_blocked(A: np.ndarray, Bt: np.ndarray) -> np.ndarray:
    """Threaded, blocked fp32 GEMM against K-major Bt [N,K] (the timed CPU baseline)."""
    A = np.ascontiguousarray(A, np.float32)
    Bt = np.ascontiguousarray(Bt, np.float32)
    M, K = A.shape
    N = Bt.shape[0]
    Cm = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32_blocked(_p(A), _sz(K), _p(Bt), _sz(K), _p(Cm), _sz(N), _sz(M), _sz(N), _sz(K))
    return Cm


def gemm_i8_blocked(A: np.ndarray, Bt: np.ndarray) -> np.ndarray:
    A = np.ascontiguousarray(A, np.int8)
    Bt = np.ascontiguousarray(Bt, np.int8)
    M, K = A.shape
    N = Bt.shape[0]
    Cm = np.empty((M, N), np.int32)
    lib().oracle_gemm_i8_blocked(_p(A), _sz(K), _p(Bt), _sz(K), _p(Cm), _sz(N), _sz(M), _sz(N), _sz(K))
    return Cm


def gemm_fp8_block_scaled(A: np.ndarray, Bt: np.ndarray, a_scale: np.ndarray, b_scale: np.ndarray,
                          out_kind: int = OUT_F32) -> np.ndarray:
    """Block-scaled FP8 GEMM on decoded operand values: A [M,K], Bt [N,K], a_scale [ceil(K/128), M],
    b_scale [ceil(K/128), ceil(N/128)]. Returns fp32 values or bf16/fp16 bit patterns [M,N]."""
    A = np.ascontiguousarray(A, np.float32)
    Bt = np.ascontiguousarray(Bt, np.float32)
    a_scale = np.ascontiguousarray(a_scale, np.float32)
    b_scale = np.ascontiguousarray(b_scale, np.float32)
    M, K = A.shape
    N = Bt.shape[0]
    kbs, nbs = -(-K // 128), -(-N // 128)
    assert Bt.shape[1] == K and a_scale.shape == (kbs, M) and b_scale.shape == (kbs, nbs)
    out = np.empty((M, N), np.float32 if out_kind == OUT_F32 else np.uint16)
    lib().oracle_gemm_fp8_block_scaled(_p(A), _sz(K), _p(Bt), _sz(K), _p(a_scale), _p(b_scale), _p(out), _sz(N),
                                       _sz(M), _sz(N), _sz(K), C.c_int(out_kind))
    return out


def scale_cast(acc: np.ndarray, sA: float, sB: float, out_kind: int) -> np.ndarray:
    """out = cast(sA*sB*acc): fp32 values, or bf16 / fp16 bit patterns."""
    acc = np.ascontiguousarray(acc)
    out = np.empty(acc.shape, np.float32 if out_kind == OUT_F32 else np.uint16)
    fn = lib().oracle_scale_cast_i32 if acc.dtype == np.int32 else lib().oracle_scale_cast_f32
    assert acc.dtype in (np.int32, np.float32)
    fn(_p(acc), _sz(acc.size), C.c_float(sA), C.c_float(sB), C.c_int(out_kind), _p(out))
    return out


def transpose(x: np.ndarray) -> np.ndarray:
    """out[c, r] = in[r, c] for any 1/2/4-byte element type."""
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    out = np.empty((cols, rows), x.dtype)
    lib().oracle_transpose(_p(x), _p(out), _sz(rows), _sz(cols), _sz(cols), _sz(rows), _sz(x.dtype.itemsize))
    return out


def harness_fill(n: int, which_b: bool) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().oracle_harness_fill(_p(out), _sz(n), C.c_int(int(which_b)))
    return out


# ---------------------------------------------------------------- error metrics
def rel_l2(c: np.ndarray, ref: np.ndarray) -> float:
    c = c.astype(np.float64).ravel()
    ref = ref.astype(np.float64).ravel()
    den = np.linalg.norm(ref)
    return float(np.linalg.norm(c - ref) / (den if den > 0 else 1.0))


def max_rel(c: np.ndarray, ref: np.ndarray, eps: float = 1e-2) -> float:
    """max |c-ref| / max(|ref|, eps*rms(ref)): element-wise relative error with a floor, since a
    pure relative error is unbounded where the reference crosses zero."""
    c = c.astype(np.float64).ravel()
    ref = ref.astype(np.float64).ravel()
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    den = np.maximum(np.abs(ref), max(eps * rms, 1e-30))
    return float(np.max(np.abs(c - ref) / den)) if ref.size else 0.0


def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> int:
    """Largest distance, in bf16 units in the last place, between two arrays of bf16 bit patterns."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    if a_bits.size == 0:
        return 0
    return int(np.max(np.abs(key(a_bits) - key(b_bits))))
