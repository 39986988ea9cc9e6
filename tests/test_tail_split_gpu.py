"""The last-wave split of the CTA-pair kernel: when the number of 256 x 256 (or 256 x 128) tiles leaves a short last wave, those
tiles' K ranges are cut into slices over all clusters (a second launch writing 32-bit partial sums into scratch
slots) and added up by a small third kernel. Shapes here are chosen so that it triggers on a 148-SM part (74
clusters): 10 x 8 = 80 tiles -> 6 tiles in the last wave, and K deep enough for the saving to beat the extra launch. Parity tiers as for the ordinary path: int8 exact,
16-bit inputs rel-L2 <= 1e-3 against the fp32 oracle; and the split must not change a result beyond the
rounding of a different summation order."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def _pair(q):
    # CTA pairs forced, everything else (and with it the last-wave split) left to the library
    return q.Tuning(0, 0, 0, 0, 1, 0)


def _no_split(q):
    return q.Tuning(0, 1, 0, 0, 1, 0)  # an explicit split_k = 1 turns the last-wave split off


def _status_ok(q):
    rc, st = q.device_status()
    assert rc == 0, f"device status {st}"


@pytest.mark.parametrize("M,N,K", [(2560, 2048, 16384), (2500, 2000, 16400), (1280, 3840, 12288)])
def test_int8_exact_with_last_wave_split(qlib, oracle, dev, M, N, K):
    q = qlib
    need = q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _pair(q))
    assert need > 0, "the shape was meant to trigger the last-wave split (scratch for its partial sums)"
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _no_split(q)) == 0
    ai = datagen.int8_uniform((M, K), seed=K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    ref = torch.full((M, N), -2, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_pair(q))
    q.gemm(a, b, ref, b_kmajor=True, tuning=_no_split(q))
    _status_ok(q)
    assert torch.equal(acc, ref), "the split and the unsplit kernel must agree exactly"
    # the CPU oracle on bands of rows: the first rows (full waves) and the last (the last wave's tiles live there)
    got = acc.cpu().numpy()
    for m0, m1 in ((0, 8), (M // 2, M // 2 + 8), (M - 264, M - 256), (M - 8, M)):
        assert np.array_equal(got[m0:m1], oracle.gemm_i8_rows(ai, bi, m0, m1))
    # scaled 16-bit output: identical to the unsplit kernel's (the accumulator is exact either way)
    sa, sb = torch.tensor([0.013], device=dev), torch.tensor([0.009], device=dev)
    c1 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    c2 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, sa, sb, c1, b_kmajor=True, tuning=_pair(q))
    q.mix_gemm(a, b, sa, sb, c2, b_kmajor=True, tuning=_no_split(q))
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
    _status_ok(q)


def test_shallow_k_keeps_the_single_launch(qlib):
    """The split costs a launch and a pass over 32-bit partial sums: with few K blocks to save it is not taken."""
    q = qlib
    assert q.workspace_query(q.BF16, q.B_K_MAJOR, 4096, 4096, 4096, _pair(q)) == 0
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, 2560, 2048, 2048, _pair(q)) == 0
    assert q.workspace_query(q.BF16, q.B_K_MAJOR, 8192, 8192, 8192, _pair(q)) == 0  # 62 of 74 in the last wave


@pytest.mark.parametrize("b_kmajor", [True, False])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_bf16_with_last_wave_split(qlib, oracle, dev, b_kmajor, out_dtype):
    q = qlib
    M, N, K = 2560, 2048, 8192
    assert q.workspace_query(q.BF16, q.B_K_MAJOR, M, N, K, _pair(q)) > 0
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=3, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K) if b_kmajor else (K, N), seed=3, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
    q.gemm(a, b, c, b_kmajor=b_kmajor, tuning=_pair(q))
    _status_ok(q)
    got = c.float().cpu().numpy()
    ref = oracle.gemm_f32(a_val, b_val, b_kmajor)
    assert np.isfinite(got).all()
    assert oracle.rel_l2(got, ref) <= (1e-3 if out_dtype == torch.float32 else 4e-3)
    # against the unsplit kernel: the tiles of the full waves are bit-identical, the last wave's differ only by
    # the order of the fp32 additions
    c0 = torch.empty_like(c)
    q.gemm(a, b, c0, b_kmajor=b_kmajor, tuning=_no_split(q))
    diff = (c.float() - c0.float()).abs().max().item()
    scale = c0.float().abs().max().item()
    assert diff <= scale * (2.0 ** -7 if out_dtype == torch.bfloat16 else 1e-5)
    changed = int((c.view(torch.int32 if out_dtype == torch.float32 else torch.int16) !=
                   c0.view(torch.int32 if out_dtype == torch.float32 else torch.int16)).any(dim=1).sum().item())
    assert changed <= 6 * 256, "only rows of the six last-wave tiles may differ"


def test_fp8_scaled_with_last_wave_split(qlib, oracle, dev):
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no float8 dtype in this torch")
    q = qlib
    M, N, K = 2560, 2048, 16384
    assert q.workspace_query(q.FP8_E4M3, q.B_K_MAJOR, M, N, K, _pair(q)) > 0
    a_bits, a_val, sa = oracle.quantize_e4m3(datagen.normal((M, K), seed=8, stream=0))
    b_bits, b_val, sb = oracle.quantize_e4m3(datagen.normal((N, K), seed=8, stream=1))
    a = torch.from_numpy(a_bits).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b_bits).to(dev).view(torch.float8_e4m3fn)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c, b_kmajor=True, tuning=_pair(q))
    _status_ok(q)
    ref = oracle.gemm_f32_blocked(a_val, b_val) * (np.float32(sa) * np.float32(sb))
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= 1e-2


def test_unaligned_c_falls_back_to_the_unsplit_kernel(qlib, oracle, dev):
    """A C that cannot take TMA stores keeps the single-launch path (the plan had reserved scratch for the split);
    the result is still exact."""
    q = qlib
    M, N, K = 2560, 2047, 16384
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _pair(q)) > 0
    ai = datagen.int8_uniform((M, K), seed=1, stream=0)
    bi = datagen.int8_uniform((N, K), seed=1, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_pair(q))
    got = acc.cpu().numpy()
    for m0, m1 in ((0, 8), (M - 8, M)):
        assert np.array_equal(got[m0:m1], oracle.gemm_i8_rows(ai, bi, m0, m1))
    _status_ok(q)


# ---- the same split with 256 x 128 pair tiles (80 tiles on 74 clusters: six tiles in the last wave)

def _narrow(q):
    return q.Tuning(128, 0, 0, 0, 1, 0)


def _narrow_no_split(q):
    return q.Tuning(128, 1, 0, 0, 1, 0)


# 80 tiles (one wave and six tiles), ragged, a single-row-of-tiles-free shape, and 160 tiles (two waves and twelve)
@pytest.mark.parametrize("M,N,K,tail", [(1280, 2048, 8192, 6), (1250, 2000, 8208, 6), (512, 5120, 12288, 6),
                                        (2560, 2048, 8192, 12)])
def test_int8_exact_with_last_wave_split_of_narrow_pair_tiles(qlib, oracle, dev, M, N, K, tail):
    q = qlib
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _narrow(q))
    assert (plan["tile_m"], plan["tile_n"], plan["ctas_per_tile"], plan["tail_tiles"]) == (256, 128, 2, tail), plan
    assert plan["tail_slices"] >= 2
    need = q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _narrow(q))
    assert need == plan["tail_slices"] * tail * 256 * 128 * 4
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _narrow_no_split(q)) == 0
    ai = datagen.int8_uniform((M, K), seed=K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    ref = torch.full((M, N), -2, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_narrow(q))
    q.gemm(a, b, ref, b_kmajor=True, tuning=_narrow_no_split(q))
    _status_ok(q)
    assert torch.equal(acc, ref), "the split and the unsplit kernel must agree exactly"
    got = acc.cpu().numpy()
    for m0, m1 in ((0, 8), (M // 2, M // 2 + 8), (M - 8, M)):
        assert np.array_equal(got[m0:m1], oracle.gemm_i8_rows(ai, bi, m0, m1))
    sa, sb = torch.tensor([0.013], device=dev), torch.tensor([0.009], device=dev)
    c1 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    c2 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, sa, sb, c1, b_kmajor=True, tuning=_narrow(q))
    q.mix_gemm(a, b, sa, sb, c2, b_kmajor=True, tuning=_narrow_no_split(q))
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
    _status_ok(q)


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_float_kinds_with_last_wave_split_of_narrow_pair_tiles(qlib, oracle, dev, kind):
    q = qlib
    M, N, K = 512, 5120, 5120 if kind == "bf16" else 8192
    dt = q.BF16 if kind == "bf16" else q.FP8_E4M3
    # the planner's own choice for this shape: 80 tiles of 256 x 128, the last six in K slices
    plan = q.plan_query(dt, q.BF16, q.B_K_MAJOR, M, N, K)
    assert (plan["tile_m"], plan["tile_n"], plan["ctas_per_tile"], plan["tail_tiles"]) == (256, 128, 2, 6), plan
    a32, b32 = datagen.normal((M, K), 5, 0), datagen.normal((N, K), 5, 1)
    tdt = torch.bfloat16 if kind == "bf16" else torch.float8_e4m3fn
    a, b = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    for out in (torch.float32, torch.bfloat16):
        c = torch.full((M, N), float("nan"), dtype=out, device=dev)
        q.gemm(a, b, c, b_kmajor=True)
        got = c.float().cpu().numpy()
        assert np.isfinite(got).all()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if out == torch.float32 else 4e-3)  # 16-bit tier
        c0 = torch.empty_like(c)
        q.gemm(a, b, c0, b_kmajor=True, tuning=_narrow_no_split(q))
        view = torch.int32 if out == torch.float32 else torch.int16
        changed = int((c.view(view) != c0.view(view)).any(dim=1).sum().item())
        assert changed <= 6 * 256, "only rows of the six last-wave tiles may differ"
    _status_ok(q)
