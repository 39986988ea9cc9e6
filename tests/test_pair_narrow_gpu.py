"""256 x 128 tiles on CTA pairs (gemm_tcgen05_pair_kernel<..., BN = 128>): each CTA of the pair loads 128 rows of A and
its 64-row half of the B tile. Same sums as every other tiling of the same K order, so int8 must agree bit for bit
with the oracle and with the lone 128 x 128 tiles; floating-point kinds are checked at their tier. Taken by the
planner for mid-size problems whose 256 x 128 tiles run in one wave; forced here with tile_n = 128, cta_pair = 1."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

# one tile; ragged M, N and K; several tiles; an unaligned C (register stores); more tiles than clusters (persistent loop)
SHAPES = [(256, 128, 512), (300, 203, 1040), (1024, 2048, 2048), (130, 520, 272), (2304, 2176, 384)]


def _narrow(q, split=1):
    return q.Tuning(128, split, 0, 0, 1, 0)


@pytest.mark.parametrize("split", [1, 2, 3])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int8_exact_and_scaled(qlib, oracle, dev, M, N, K, split):
    q = qlib
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _narrow(q, split))
    assert (plan["tile_m"], plan["tile_n"], plan["ctas_per_tile"]) == (256, 128, 2), plan
    ai = datagen.int8_uniform((M, K), seed=M + N, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + N, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_narrow(q, split))
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref)
    lone = torch.full((M, N), -8, dtype=torch.int32, device=dev)
    q.gemm(a, b, lone, b_kmajor=True, tuning=q.Tuning(128, 1, 0, 0, -1, 0))
    assert torch.equal(acc, lone)
    sa, sb = datagen.scale_pair(5)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, c, b_kmajor=True, tuning=_narrow(q, split))
    bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(bits, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("kind", ["bf16", "fp16", "fp8"])
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_float_kinds(qlib, oracle, dev, M, N, K, kind):
    q = qlib
    a32, b32 = datagen.normal((M, K), M + K, 0), datagen.normal((N, K), M + K, 1)
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": torch.float8_e4m3fn}[kind]
    a, b = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    for dt in (torch.float32, torch.bfloat16):
        c = torch.full((M, N), -3, dtype=dt, device=dev)
        q.gemm(a, b, c, b_kmajor=True, tuning=_narrow(q))
        got = c.float().cpu().numpy()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier: max relative error with an rms floor
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if dt == torch.float32 else 4e-3)  # 16-bit tier
    rc, st = q.device_status()
    assert rc == 0, st


def test_planner_takes_narrow_pairs_for_one_wave_of_mid_size_tiles(qlib):
    q = qlib
    for dt in (q.BF16, q.FP8_E4M3):
        p = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 1024, 2048, 8192)
        assert (p["tile_m"], p["tile_n"], p["ctas_per_tile"], p["split_k"], p["ctas"]) == (256, 128, 2, 1, 128), p
        big = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 4096, 4096, 4096)  # several waves: 256 x 256 pairs
        assert (big["tile_m"], big["tile_n"]) == (256, 256), big


def test_failure_detection_on_narrow_pair(qlib, oracle, dev):
    """The host-made failure of test_failure_detection_gpu.py on one 256 x 128 tile: the pair leaves together."""
    q = qlib
    M, N, K = 256, 128, 512
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=8, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=8, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=True, tuning=_narrow(q))
    assert q.device_status()[0] == q.OK
    q.lib().qgemm_test_arm_skip_load(3)
    q.gemm(a, b, c, b_kmajor=True, tuning=_narrow(q))
    rc, st = q.device_status()
    assert rc == q.ERR_DEVICE_TIMEOUT and st[0] == 1 and st[1] == 0 and st[2] == 2 and st[3] == 3, st
    q.gemm(a, b, c, b_kmajor=True, tuning=_narrow(q))
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK
