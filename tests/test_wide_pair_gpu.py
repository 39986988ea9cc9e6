"""The wide CTA-pair kernel (512 x 256 tiles per cluster of two, both accumulators of a CTA in use): same results as
the 256 x 256 pair kernel, bit for bit (every element is the same sum in the same order), on whole, ragged and small
shapes, for every input kind; int8 also against the CPU oracle."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def _tunings(q):
    return q.Tuning(0, 1, 0, 0, 2, 0), q.Tuning(0, 1, 0, 0, 1, 0)  # wide, 256 x 256 pairs (no split either way)


@pytest.mark.parametrize("M,N,K", [(512, 256, 128), (1024, 512, 256), (600, 300, 200), (2048, 2048, 1024),
                                    (130, 70, 72), (4096, 1024, 512), (1537, 769, 264)])
@pytest.mark.parametrize("b_kmajor", [True, False])
def test_bf16_matches_the_pair_kernel_and_the_oracle(qlib, oracle, dev, M, N, K, b_kmajor):
    q = qlib
    wide, pair = _tunings(q)
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=M + K, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K) if b_kmajor else (K, N), seed=M + K, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    if not b_kmajor and (N * 2) % 16 != 0:
        pytest.skip("row-major B with an unaligned leading dimension goes through the relayout, covered elsewhere")
    for out_dtype in (torch.float32, torch.bfloat16):
        cw = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
        cp = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev)
        q.gemm(a, b, cw, b_kmajor=b_kmajor, tuning=wide)
        q.gemm(a, b, cp, b_kmajor=b_kmajor, tuning=pair)
        rc, st = q.device_status()
        assert rc == 0, st
        assert torch.equal(cw.view(torch.int32 if out_dtype == torch.float32 else torch.int16),
                           cp.view(torch.int32 if out_dtype == torch.float32 else torch.int16))
    assert oracle.rel_l2(cw.float().cpu().numpy(), oracle.gemm_f32(a_val, b_val, b_kmajor)) <= 4e-3
    q.gemm(a, b, c32 := torch.zeros((M, N), dtype=torch.float32, device=dev), b_kmajor=b_kmajor, tuning=wide)
    assert oracle.rel_l2(c32.cpu().numpy(), oracle.gemm_f32(a_val, b_val, b_kmajor)) <= 1e-3


@pytest.mark.parametrize("M,N,K", [(1024, 768, 512), (700, 520, 1040), (2304, 1280, 2048)])
def test_int8_exact_and_scaled(qlib, oracle, dev, M, N, K):
    q = qlib
    wide, pair = _tunings(q)
    ai = datagen.int8_uniform((M, K), seed=K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=wide)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, True))
    sa, sb = torch.tensor([0.004], device=dev), torch.tensor([0.007], device=dev)
    cw = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    cp = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, sa, sb, cw, b_kmajor=True, tuning=wide)
    q.mix_gemm(a, b, sa, sb, cp, b_kmajor=True, tuning=pair)
    assert torch.equal(cw.view(torch.int16), cp.view(torch.int16))
    rc, st = q.device_status()
    assert rc == 0, st


def test_fp8_matches_the_pair_kernel(qlib, oracle, dev):
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no float8 dtype in this torch")
    q = qlib
    wide, pair = _tunings(q)
    M, N, K = 1536, 1024, 2048
    a_bits, a_val, sa = oracle.quantize_e4m3(datagen.normal((M, K), seed=5, stream=0))
    b_bits, b_val, sb = oracle.quantize_e4m3(datagen.normal((N, K), seed=5, stream=1))
    a = torch.from_numpy(a_bits).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b_bits).to(dev).view(torch.float8_e4m3fn)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    cw = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    cp = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, cw, b_kmajor=True, tuning=wide)
    q.mix_gemm(a, b, tsa, tsb, cp, b_kmajor=True, tuning=pair)
    assert torch.equal(cw.view(torch.int16), cp.view(torch.int16))
    ref = oracle.gemm_f32_blocked(a_val, b_val) * (np.float32(sa) * np.float32(sb))
    assert oracle.max_rel(cw.float().cpu().numpy(), ref) <= 1e-2


def test_unaligned_c_takes_the_ordinary_pairs(qlib, oracle, dev):
    q = qlib
    wide, _ = _tunings(q)
    M, N, K = 520, 263, 128  # N odd: C cannot be stored through TMA
    ai = datagen.int8_uniform((M, K), seed=9, stream=0)
    bi = datagen.int8_uniform((N, K), seed=9, stream=1)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.gemm(torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev), acc, b_kmajor=True, tuning=wide)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, True))


def test_when_the_library_takes_wide_tiles_by_itself(qlib):
    """16-bit inputs, deep K and at least six waves of 512 x 256 tiles; never for the 8-bit kinds."""
    q = qlib
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192)["tile_m"] == 512
    assert q.plan_query(q.FP16, q.FP32, q.B_K_MAJOR, 16384, 8192, 8192)["tile_m"] == 512
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 4096, 4096, 4096)["tile_m"] == 256
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 6144, 7168, 8192)["tile_m"] == 256
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 8192, 8192, 4096)["tile_m"] == 256
    assert q.plan_query(q.INT8, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192)["tile_m"] == 256
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192)["tile_m"] == 256
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192, q.Tuning(0, 0, 0, 0, 1, 0))["tile_m"] == 256
