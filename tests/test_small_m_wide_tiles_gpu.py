"""Small M on the 128- and 256-wide lone tiles: the kernels load only 16 / 32 / 64 rows of A per stage (32 / 16 with the
256-wide tile) while the MMA still reads 128 rows; whatever lies behind the loaded rows must reach no stored element.
Same K order as every other tiling, so int8 must agree bit for bit with the oracle and with the full-box form of the
same tile (QGEMM_FULL_A_TILE=1); floating-point kinds are checked at their tier. Shapes cover every row class, ragged
N and K, several tiles per CTA (persistent loop), K slices in two launches and inside one cluster, and row-major B."""
import os

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

# (M, N, K): M = 1, 16 | 17, 32 | 33, 64 (the three row classes and their edges)
# (16, 512, 640): five K blocks of int8, an odd count for the two-blocks-per-load form of the 128-wide tile on 16 rows
SHAPES = [(1, 384, 512), (16, 1000, 1040), (17, 640, 272), (32, 2304, 384), (33, 520, 2048), (64, 203, 768),
          (8, 40000, 256), (16, 512, 640)]


def _rows(M, bn):
    if bn == 256:
        return 16 if M <= 16 else (32 if M <= 32 else 128)
    return 16 if M <= 16 else (32 if M <= 32 else 64)


def _tune(q, bn, split=1):
    return q.Tuning(bn, split, 0, 0, -1, 0)


@pytest.mark.parametrize("split", [1, 3])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int8_exact_and_scaled(qlib, oracle, dev, M, N, K, bn, split):
    q = qlib
    if split > K // 128:
        pytest.skip("fewer K blocks than slices")
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _tune(q, bn, split))
    assert (plan["tile_m"], plan["tile_n"], plan["ctas_per_tile"], plan["a_rows_per_stage"]) == (128, bn, 1, _rows(M, bn)), plan
    ai = datagen.int8_uniform((M, K), seed=M + N, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + N, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_tune(q, bn, split))
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref)
    os.environ["QGEMM_FULL_A_TILE"] = "1"
    try:
        q.lib().qgemm_reload_env()
        full_plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _tune(q, bn, split))
        assert full_plan["a_rows_per_stage"] == 128, full_plan
        full = torch.full((M, N), -8, dtype=torch.int32, device=dev)
        q.gemm(a, b, full, b_kmajor=True, tuning=_tune(q, bn, split))
    finally:
        del os.environ["QGEMM_FULL_A_TILE"]
        q.lib().qgemm_reload_env()
    assert torch.equal(acc, full)
    sa, sb = datagen.scale_pair(5)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, c, b_kmajor=True, tuning=_tune(q, bn, split))
    bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(bits, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8"])
@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("M,N,K", SHAPES[:6] + SHAPES[7:])
def test_float_kinds(qlib, oracle, dev, M, N, K, bn, kind):
    q = qlib
    a32, b32 = datagen.normal((M, K), M + K, 0), datagen.normal((N, K), M + K, 1)
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}[kind]
    a, b = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    for dt in (torch.float32, torch.bfloat16):
        c = torch.full((M, N), -3, dtype=dt, device=dev)
        q.gemm(a, b, c, b_kmajor=True, tuning=_tune(q, bn))
        got = c.float().cpu().numpy()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier: max relative error with an rms floor
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if dt == torch.float32 else 4e-3)  # 16-bit tier
    rc, st = q.device_status()
    assert rc == 0, st


# K a multiple of 8 x 128 bytes, so that 2, 4 and 8 slices are all non-empty and equal
# (16, 256, 3072): three K blocks per slice with eight slices, an odd count for the two-blocks-per-load form
CLUSTER_SHAPES = [(1, 384, 2048), (16, 1000, 2048), (17, 640, 4096), (33, 520, 2048), (64, 203, 3072), (16, 256, 3072)]


@pytest.mark.parametrize("slices", [2, 4, 8])
@pytest.mark.parametrize("M,N,K", CLUSTER_SHAPES)
def test_in_cluster_split_k_on_128_wide_tiles(qlib, oracle, dev, M, N, K, slices):
    """The K slices of a 128-wide tile on the CTAs of one cluster, 16 / 32 / 64 rows of A per stage: int8 bit for bit
    against the oracle and against the two-launch split at the same slice count; BF16 and FP8 at their tiers."""
    q = qlib
    tun = q.Tuning(128, slices, 0, 0, -1, 0)
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, tun)
    assert (plan["tile_n"], plan["split_k"], plan["cluster_slices"], plan["a_rows_per_stage"]) == (128, slices, slices, _rows(M, 128)), plan
    ai = datagen.int8_uniform((M, K), seed=M + N, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + N, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=tun)
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref)
    sa, sb = datagen.scale_pair(5)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, c, b_kmajor=True, tuning=tun)
    os.environ["QGEMM_KCLUSTER"] = "0"
    try:
        q.lib().qgemm_reload_env()
        assert q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, tun)["cluster_slices"] == 0
        c2 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
        q.mix_gemm(a, b, tsa, tsb, c2, b_kmajor=True, tuning=tun)
    finally:
        del os.environ["QGEMM_KCLUSTER"]
        q.lib().qgemm_reload_env()
    assert torch.equal(c.view(torch.int16), c2.view(torch.int16))  # same sums in the same order, same scale and cast
    bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(bits, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1
    for kind, tdt in (("bf16", torch.bfloat16), ("fp8", torch.float8_e4m3fn)):
        a32, b32 = datagen.normal((M, K), M + K, 0), datagen.normal((N, K), M + K, 1)
        fa, fb = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
        fref = oracle.gemm_f32(fa.float().numpy(), fb.float().numpy(), True)
        out = torch.full((M, N), -3, dtype=torch.float32, device=dev)
        q.gemm(fa.to(dev), fb.to(dev), out, b_kmajor=True, tuning=tun)
        got = out.cpu().numpy()
        if kind == "fp8":
            assert oracle.max_rel(got, fref) <= 1e-2  # fp8 tier
        else:
            assert oracle.rel_l2(got, fref) <= 1e-3  # 16-bit tier, fp32 out
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("bn", [128, 256])
def test_row_major_b_int8(qlib, oracle, dev, bn):
    """B as the reference lays it out ([K, N] row-major), read in place and through the relayout pre-pass."""
    q = qlib
    M, N, K = 16, 768, 640
    ai = datagen.int8_uniform((M, K), seed=21, stream=0)
    bi = datagen.int8_uniform((K, N), seed=21, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    ref = oracle.gemm_i8(ai, bi, False)
    for relayout in (0, 1):
        acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
        q.gemm(a, b, acc, b_kmajor=False, tuning=q.Tuning(bn, 1, 0, 0, -1, relayout))
        assert np.array_equal(acc.cpu().numpy(), ref), relayout
    assert q.device_status()[0] == q.OK


def test_planner_rows_per_stage(qlib):
    q = qlib
    # two K blocks per TMA instruction with the 128-wide tile only on 16 rows of A (slices inside a cluster included)
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 11008, 4096)["k_blocks_per_load"] == 2
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 32, 11008, 4096)["k_blocks_per_load"] == 1
    assert q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, 16, 1000, 2048, q.Tuning(128, 4, 0, 0, -1, 0))["k_blocks_per_load"] == 2
    assert q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, 17, 640, 4096, q.Tuning(128, 4, 0, 0, -1, 0))["k_blocks_per_load"] == 1
    # a skinny problem whose 64-wide tiles would need two waves: one wave of 128-wide tiles on 16 rows of A
    p = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 11008, 4096)
    assert (p["tile_n"], p["split_k"], p["a_rows_per_stage"], p["ctas"]) == (128, 1, 16, 86), p
    p = q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 1, 28672, 8192)
    assert (p["tile_n"], p["a_rows_per_stage"]) == (256, 16), p
    p = q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 48, 28672, 8192)
    assert (p["tile_n"], p["a_rows_per_stage"]) == (256, 128), p
