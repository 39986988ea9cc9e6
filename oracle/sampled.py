"""Sampled parity checks of a GPU result against the CPU oracle, for problems too large to check whole.

Test infrastructure, like the rest of this directory: used by tests/ and by bench.py's `oracle_check` (outside
every timed region), never by the product path. A full-size product (8192^3 and beyond) is checked on a few row
bands -- the first rows, rows straddling an output-tile edge, and the last rows -- over all columns, or over
chosen column windows; int32 sampling stays bit-exact, the other tiers keep their tolerance:

    int8 -> int32   bit-exact
    int8 -> bf16    <= 1 bf16 ulp of bf16(sA * sB * float(acc))      (README.md:5-7 of the reference)
    fp8  -> any     max |c - ref| / max(|ref|, 1e-2 rms(ref)) <= 1e-2 against fp32 accumulation
    fp16 / bf16     rel-L2 <= 1e-3 against fp32 accumulation (+ the rounding of a 16-bit output, 4e-3)
    block-scaled fp8 (src/mix_gemm/hip_mix_gemm_kernel.cpp:193-244): as the fp8 tier

Every function takes `fetch(m0, m1)`, which returns rows [m0, m1) of the GPU result as a numpy array (values for
floating-point outputs, uint16 bit patterns where stated), so that only the sampled rows leave the device.
"""
from __future__ import annotations

import numpy as np

from . import oracle as o

REL_L2_TOL = 1e-3
REL_L2_TOL_16BIT_OUT = 4e-3
FP8_MAX_REL_TOL = 1e-2
BF16_ULP_TOL = 1


def row_bands(M: int, rows: int = 12, tile: int = 256):
    """Starts of the sampled row bands: the first rows, a band straddling an output-tile edge near the middle, the
    last rows (fewer when M is small)."""
    rows = min(rows, M)
    mid = (M // 2) // tile * tile - rows // 2
    starts = {0, max(0, min(M - rows, mid)), M - rows}
    return sorted(starts), rows


def check_int8(A: np.ndarray, Bt: np.ndarray, fetch, out: str, sa: float = 1.0, sb: float = 1.0, rows: int = 12,
               cols=None) -> dict:
    """A [M,K], Bt [N,K] int8. out = "int32" (fetch returns int32, compared bit for bit) or "bf16" (fetch returns
    uint16 bit patterns, compared in ulps with bf16(sa*sb*acc)). `cols` = optional list of (n0, n1) column windows."""
    M = A.shape[0]
    starts, rows = row_bands(M, rows)
    windows = cols if cols else [(0, Bt.shape[0])]
    worst, exact = 0, True
    for m0 in starts:
        got = fetch(m0, m0 + rows)
        for n0, n1 in windows:
            acc = o.gemm_i8_rows(A, np.ascontiguousarray(Bt[n0:n1]), m0, m0 + rows)
            if out == "int32":
                exact = exact and bool(np.array_equal(got[:, n0:n1], acc))
            else:
                ref_bits = o.scale_cast(acc, float(sa), float(sb), o.OUT_BF16)
                worst = max(worst, o.bf16_ulp_distance(np.ascontiguousarray(got[:, n0:n1]), ref_bits))
    ok = exact if out == "int32" else worst <= BF16_ULP_TOL
    return {"tier": "int8 accumulator bit-exact" if out == "int32" else "int8 scaled output <= 1 bf16 ulp",
            "row_bands": [[m0, m0 + rows] for m0 in starts], "column_windows": [list(w) for w in windows],
            "max_bf16_ulp": None if out == "int32" else worst, "ok": bool(ok)}


def check_float(a_rows, Bt_val: np.ndarray, fetch, M: int, tier: str, scale: float = 1.0, out_16bit: bool = True,
                rows: int = 12) -> dict:
    """a_rows(m0, m1) returns rows of A as exact fp32 values; Bt_val [N,K] fp32 values. tier = "f16" (rel-L2) or
    "fp8" (max relative error with an rms floor); `scale` multiplies the fp32-accumulated reference."""
    starts, rows = row_bands(M, rows)
    worst = 0.0
    for m0 in starts:
        ref = o.gemm_f32_blocked(a_rows(m0, m0 + rows), Bt_val) * np.float32(scale)
        got = fetch(m0, m0 + rows)
        err = o.rel_l2(got, ref) if tier == "f16" else o.max_rel(got, ref)
        worst = max(worst, err)
    tol = (REL_L2_TOL_16BIT_OUT if out_16bit else REL_L2_TOL) if tier == "f16" else FP8_MAX_REL_TOL
    return {"tier": "rel-L2 vs fp32 accumulation" if tier == "f16" else "fp8 max relative error (rms floor 1e-2)",
            "row_bands": [[m0, m0 + rows] for m0 in starts], "worst": worst, "tol": tol, "ok": bool(worst <= tol)}


def check_block_scaled(a_rows, Bt_val: np.ndarray, a_scale: np.ndarray, b_scale: np.ndarray, fetch, M: int,
                       rows: int = 8) -> dict:
    """Block-scaled FP8: a_scale [ceil(K/128), M], b_scale [ceil(K/128), ceil(N/128)]; the oracle is run on the
    sampled rows with the matching columns of a_scale."""
    starts, rows = row_bands(M, rows, tile=128)
    worst = 0.0
    for m0 in starts:
        ref = o.gemm_fp8_block_scaled(a_rows(m0, m0 + rows), Bt_val, np.ascontiguousarray(a_scale[:, m0:m0 + rows]),
                                      b_scale, o.OUT_F32)
        worst = max(worst, o.max_rel(fetch(m0, m0 + rows), ref))
    return {"tier": "block-scaled fp8 max relative error (rms floor 1e-2)",
            "row_bands": [[m0, m0 + rows] for m0 in starts], "worst": worst, "tol": FP8_MAX_REL_TOL,
            "ok": bool(worst <= FP8_MAX_REL_TOL)}
