"""Split-K inside one launch (gemm_sm100_kcluster.cuh): the K slices of a 64- or 128-wide tile run on the CTAs of one
cluster, and the partial sums are added up through distributed shared memory in slice order -- the order in which
splitk_reduce_kernel adds the slabs of the two-launch form. So the two forms must agree BIT FOR BIT for every input
type, and both are checked against the oracle at their tier. QGEMM_KCLUSTER=0 (read when the library reads its
environment) selects the two-launch form for the comparison."""
import os

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

# M, N, K: one tile row / several, ragged M and N (N = 516: rows that are 16-byte multiples for 32-bit outputs only;
# N = 203: register stores column by column), K not a multiple of the slices' block count
SHAPES = [(32, 2048, 8192), (16, 1024, 4096), (100, 516, 3008), (300, 203, 2064), (128, 64, 256), (1, 8, 272)]


def _two_launch(q, fn):
    os.environ["QGEMM_KCLUSTER"] = "0"
    q.lib().qgemm_reload_env()
    try:
        return fn()
    finally:
        del os.environ["QGEMM_KCLUSTER"]
        q.lib().qgemm_reload_env()


def _tuning(q, slices, bn=64):
    return q.Tuning(bn, slices, 0, 0, -1, 0)


def _expect_cluster(q, in_dt, out_dt, M, N, K, slices, bn=64):
    """Whether the one-launch form applies: the slices must be non-empty and the clusters fit the SMs in one wave."""
    elem = 2 if in_dt in (q.BF16, q.FP16) else 1
    kb = -(-K // (128 // elem))
    kbps = -(-kb // slices)
    real = -(-kb // kbps)
    tiles = -(-M // 128) * -(-N // bn)
    plan = q.plan_query(in_dt, out_dt, q.B_K_MAJOR, M, N, K, _tuning(q, slices, bn))
    assert plan["tile_n"] == bn
    # how many clusters run at once is the device's answer (a cluster's CTAs share a GPC): well below the SM count the
    # one-launch form must be taken, above it it cannot be
    if real != slices or tiles * slices > 148:
        want = 0
    elif tiles * slices <= 64:
        want = slices
    else:
        want = plan["cluster_slices"]
        assert want in (0, slices), plan
    assert plan["cluster_slices"] == want, (plan, want)
    assert _two_launch(q, lambda: q.plan_query(in_dt, out_dt, q.B_K_MAJOR, M, N, K, _tuning(q, slices, bn)))[
        "cluster_slices"] == 0
    return want


@pytest.mark.parametrize("bn", [64, 128])
@pytest.mark.parametrize("slices", [2, 4, 8])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int8_accumulator_and_scaled_output(qlib, oracle, dev, M, N, K, slices, bn):
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=M + K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    _expect_cluster(q, q.INT8, q.INT32, M, N, K, slices, bn)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_tuning(q, slices, bn))
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref)
    sa, sb = datagen.scale_pair(3)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        c1 = torch.full((M, N), -3, dtype=dt, device=dev)
        c2 = torch.full((M, N), -4, dtype=dt, device=dev)
        q.mix_gemm(a, b, tsa, tsb, c1, b_kmajor=True, tuning=_tuning(q, slices, bn))
        _two_launch(q, lambda: q.mix_gemm(a, b, tsa, tsb, c2, b_kmajor=True, tuning=_tuning(q, slices, bn)))
        assert torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)), dt
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, c, b_kmajor=True, tuning=_tuning(q, slices, bn))
    bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(bits, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("bn", [64, 128])
@pytest.mark.parametrize("slices", [2, 4, 8])
@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_float_kinds_match_two_launch_form_bit_for_bit(qlib, oracle, dev, M, N, K, kind, slices, bn):
    q = qlib
    a32, b32 = datagen.normal((M, K), M + N, 0), datagen.normal((N, K), M + N, 1)
    if kind == "fp8":
        a = torch.from_numpy(a32).to(torch.float8_e4m3fn)
        b = torch.from_numpy(b32).to(torch.float8_e4m3fn)
        in_dt = q.FP8_E4M3
    else:
        tdt = torch.bfloat16 if kind == "bf16" else torch.float16
        a, b = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
        in_dt = q.BF16 if kind == "bf16" else q.FP16
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    _expect_cluster(q, in_dt, q.FP32, M, N, K, slices, bn)
    for dt in (torch.float32, torch.bfloat16):
        c1 = torch.full((M, N), -3, dtype=dt, device=dev)
        c2 = torch.full((M, N), -4, dtype=dt, device=dev)
        q.gemm(a, b, c1, b_kmajor=True, tuning=_tuning(q, slices, bn))
        _two_launch(q, lambda: q.gemm(a, b, c2, b_kmajor=True, tuning=_tuning(q, slices, bn)))
        assert torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)), dt
        got = c1.float().cpu().numpy()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier: max relative error with an rms floor
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if dt == torch.float32 else 4e-3)  # 16-bit tier
    rc, st = q.device_status()
    assert rc == 0, st


def test_leading_dimensions_and_unaligned_output(qlib, oracle, dev):
    """C inside a wider buffer whose rows are not 16-byte multiples (register stores), A and B with padded rows."""
    q = qlib
    M, N, K, slices = 40, 136, 1024, 4
    ai = datagen.int8_uniform((M, K + 16), seed=9, stream=0)
    bi = datagen.int8_uniform((N, K + 32), seed=9, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    buf = torch.full((M, N + 3), -9, dtype=torch.int32, device=dev)
    c = buf[:, 1:N + 1]
    assert q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _tuning(q, slices))["cluster_slices"] == slices
    q.gemm(a[:, :K], b[:, :K], c, b_kmajor=True, tuning=_tuning(q, slices))
    assert np.array_equal(c.cpu().numpy(), oracle.gemm_i8(np.ascontiguousarray(ai[:, :K]),
                                                          np.ascontiguousarray(bi[:, :K]), True))
    assert bool((buf[:, 0] == -9).all()) and bool((buf[:, N + 1:] == -9).all())  # nothing written outside C
    assert q.device_status()[0] == q.OK


def test_cluster_leaves_together_when_a_wait_runs_out(qlib, oracle, dev):
    """The host-made failure of test_failure_detection_gpu.py on a cluster of four: the producer of every CTA leaves
    out K block 2, which only the CTA of slice 1 (K blocks 2 and 3 of 8) would have loaded; its MMA issuer's wait runs
    out, it raises the abort flag of the three other CTAs through distributed shared memory, and all four meet at the
    cluster barriers and return. The context stays usable."""
    import time
    q = qlib
    M, N, K, slices = 64, 64, 512, 4  # one tile, 8 K blocks of bf16, 2 per slice
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=5, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=5, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    t = _tuning(q, slices)
    assert q.plan_query(q.BF16, q.FP32, q.B_K_MAJOR, M, N, K, t)["cluster_slices"] == slices
    q.gemm(a, b, c, b_kmajor=True, tuning=t)  # warm
    assert q.device_status()[0] == q.OK
    q.lib().qgemm_test_arm_skip_load(2)
    t0 = time.perf_counter()
    q.gemm(a, b, c, b_kmajor=True, tuning=t)
    rc, st = q.device_status()
    elapsed = time.perf_counter() - t0
    assert rc == q.ERR_DEVICE_TIMEOUT
    code, cta, role, where = st
    assert code == 1 and cta == 1 and role == 2 and where == 2, st  # slice 1's MMA issuer, waiting for K block 2
    assert elapsed < 3.0, elapsed  # one wait limit (about a second), not the epilogue warps' doubled one on top
    assert q.device_status()[0] == q.OK
    q.gemm(a, b, c, b_kmajor=True, tuning=t)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK


# ---------------------------------------------------------------- CTA pairs: 2 or 4 pairs per cluster on a 256 x 128 tile
PAIR_SHAPES = [(256, 128, 1024), (512, 384, 2048), (300, 260, 3008), (130, 203, 2064), (1024, 512, 4096)]


def _pair_tuning(q, slices):
    return q.Tuning(128, slices, 0, 0, 1, 0)


def _expect_pair_cluster(q, in_dt, out_dt, M, N, K, slices):
    elem = 2 if in_dt in (q.BF16, q.FP16) else 1
    kb = -(-K // (128 // elem))
    kbps = -(-kb // slices)
    real = -(-kb // kbps)
    tiles = -(-M // 256) * -(-N // 128)
    plan = q.plan_query(in_dt, out_dt, q.B_K_MAJOR, M, N, K, _pair_tuning(q, slices))
    assert plan["ctas_per_tile"] == 2 and (plan["tile_m"], plan["tile_n"]) == (256, 128), plan
    if real != slices or tiles * 2 * slices > 148:
        want = 0
    elif tiles * 2 * slices <= 64:
        want = slices
    else:
        want = plan["cluster_slices"]
        assert want in (0, slices), plan
    assert plan["cluster_slices"] == want, (plan, want)
    return want


@pytest.mark.parametrize("slices", [2, 4])
@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
def test_pair_int8_accumulator_and_scaled_output(qlib, oracle, dev, M, N, K, slices):
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=M + K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    _expect_pair_cluster(q, q.INT8, q.INT32, M, N, K, slices)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_pair_tuning(q, slices))
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref)
    sa, sb = datagen.scale_pair(3)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    for dt in (torch.bfloat16, torch.float16, torch.float32):
        c1 = torch.full((M, N), -3, dtype=dt, device=dev)
        c2 = torch.full((M, N), -4, dtype=dt, device=dev)
        q.mix_gemm(a, b, tsa, tsb, c1, b_kmajor=True, tuning=_pair_tuning(q, slices))
        _two_launch(q, lambda: q.mix_gemm(a, b, tsa, tsb, c2, b_kmajor=True, tuning=_pair_tuning(q, slices)))
        assert torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)), dt
    out = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, out, b_kmajor=True, tuning=_pair_tuning(q, slices))
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(got, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("slices", [2, 4])
@pytest.mark.parametrize("kind", ["bf16", "fp8"])
@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
def test_pair_float_kinds_match_two_launch_form_bit_for_bit(qlib, oracle, dev, M, N, K, kind, slices):
    q = qlib
    a32, b32 = datagen.normal((M, K), M + N, 0), datagen.normal((N, K), M + N, 1)
    if kind == "fp8":
        a = torch.from_numpy(a32).to(torch.float8_e4m3fn)
        b = torch.from_numpy(b32).to(torch.float8_e4m3fn)
        in_dt = q.FP8_E4M3
    else:
        a, b = torch.from_numpy(a32).to(torch.bfloat16), torch.from_numpy(b32).to(torch.bfloat16)
        in_dt = q.BF16
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    _expect_pair_cluster(q, in_dt, q.FP32, M, N, K, slices)
    for dt in (torch.float32, torch.bfloat16):
        c1 = torch.full((M, N), -3, dtype=dt, device=dev)
        c2 = torch.full((M, N), -4, dtype=dt, device=dev)
        q.gemm(a, b, c1, b_kmajor=True, tuning=_pair_tuning(q, slices))
        _two_launch(q, lambda: q.gemm(a, b, c2, b_kmajor=True, tuning=_pair_tuning(q, slices)))
        assert torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)), dt
        got = c1.float().cpu().numpy()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if dt == torch.float32 else 4e-3)  # 16-bit tier
    rc, st = q.device_status()
    assert rc == 0, st


def test_pair_cluster_leaves_together_when_a_wait_runs_out(qlib, oracle, dev):
    """One 256 x 128 tile on a cluster of two pairs; K block 5 belongs to the second pair (blocks 4..7), whose leader
    is CTA 2 of the grid: its MMA issuer's wait runs out, it raises the abort flag of the three other CTAs, and all four
    meet at the cluster barriers and return."""
    import time
    q = qlib
    M, N, K, slices = 256, 128, 512, 2  # 8 K blocks of bf16, 4 per pair
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=6, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=6, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    t = _pair_tuning(q, slices)
    assert q.plan_query(q.BF16, q.FP32, q.B_K_MAJOR, M, N, K, t)["cluster_slices"] == slices
    q.gemm(a, b, c, b_kmajor=True, tuning=t)  # warm
    assert q.device_status()[0] == q.OK
    q.lib().qgemm_test_arm_skip_load(5)
    t0 = time.perf_counter()
    q.gemm(a, b, c, b_kmajor=True, tuning=t)
    rc, st = q.device_status()
    elapsed = time.perf_counter() - t0
    assert rc == q.ERR_DEVICE_TIMEOUT
    code, cta, role, where = st
    assert code == 1 and cta == 2 and role == 2 and where == 5, st
    assert elapsed < 3.0, elapsed
    assert q.device_status()[0] == q.OK
    q.gemm(a, b, c, b_kmajor=True, tuning=t)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK
