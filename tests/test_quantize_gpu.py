"""The quantisation pre-pass against the oracle: scales and quantised values bit-exact (the same IEEE
division and round-to-nearest-even on both sides), for fp32 and bf16 inputs, ragged and strided."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (128, 256), (257, 1023), (2048, 7168)])
@pytest.mark.parametrize("in_name", ["fp32", "bf16"])
def test_quantize_fp8_matches_oracle(qlib, oracle, dev, rows, cols, in_name):
    x32 = datagen.normal((rows, cols), seed=rows + cols, stream=0) * 3.0
    if in_name == "bf16":
        x32 = oracle.round_bf16(x32)[1]
    x = torch.from_numpy(x32).to(dev)
    if in_name == "bf16":
        x = x.to(torch.bfloat16)
    q8, scale = qlib.quantize(x, torch.float8_e4m3fn)
    ref_bits, _, ref_scale = oracle.quantize_e4m3(x32)
    assert float(scale.item()) == np.float32(ref_scale)
    assert np.array_equal(q8.view(torch.uint8).cpu().numpy(), ref_bits)


@pytest.mark.parametrize("rows,cols", [(1, 7), (130, 260), (1024, 4096)])
def test_quantize_int8_matches_oracle(qlib, oracle, dev, rows, cols):
    x32 = datagen.uniform((rows, cols), seed=cols, stream=1, lo=-5.0, hi=5.0)
    q8, scale = qlib.quantize(torch.from_numpy(x32).to(dev), torch.int8)
    ref_q, ref_scale = oracle.quantize_int8(x32)
    assert float(scale.item()) == np.float32(ref_scale)
    assert np.array_equal(q8.cpu().numpy(), ref_q)
    assert int(np.abs(q8.cpu().numpy().astype(np.int32)).max()) == 127


def test_quantize_strided_views_and_zero_matrix(qlib, oracle, dev):
    x32 = datagen.normal((100, 70), seed=4, stream=0)
    buf = torch.zeros((100, 96), device=dev)
    buf[:, 3:73] = torch.from_numpy(x32).to(dev)
    out = torch.full((100, 80), 0x11, dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    q8, scale = qlib.quantize(buf[:, 3:73], torch.float8_e4m3fn, out=out[:, 5:75])
    ref_bits, _, ref_scale = oracle.quantize_e4m3(x32)
    got = out.view(torch.uint8).cpu().numpy()
    assert np.array_equal(got[:, 5:75], ref_bits) and np.all(got[:, :5] == 0x11) and np.all(got[:, 75:] == 0x11)
    z, zs = qlib.quantize(torch.zeros((8, 8), device=dev), torch.int8)
    assert float(zs.item()) == 1.0 and int(z.abs().max()) == 0


def test_quantize_then_mix_gemm_end_to_end(qlib, oracle, dev):
    """fp32 operands -> quantize (device) -> FP8 mixed GEMM with the device-resident scales: close to the
    fp32 product of the unquantised operands (FP8 has 3 mantissa bits: a few percent rel-L2)."""
    M, N, K = 256, 512, 1024
    a32 = datagen.normal((M, K), seed=1, stream=0)
    b32 = datagen.normal((N, K), seed=1, stream=1)
    qa, sa = qlib.quantize(torch.from_numpy(a32).to(dev), torch.float8_e4m3fn)
    qb, sb = qlib.quantize(torch.from_numpy(b32).to(dev), torch.float8_e4m3fn)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    qlib.fp8_mm(qa, qb, sa, sb, c)
    # against the oracle on the same quantised operands: the FP8 tier
    a_val = oracle.e4m3_decode(qa.view(torch.uint8).cpu().numpy())
    b_val = oracle.e4m3_decode(qb.view(torch.uint8).cpu().numpy())
    ref = oracle.gemm_f32(a_val, b_val, True) * (np.float32(sa.item()) * np.float32(sb.item()))
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= 1e-2
    # and against the unquantised product
    assert oracle.rel_l2(c.float().cpu().numpy(), oracle.gemm_f32(a32, b32, True)) <= 6e-2


@pytest.mark.parametrize("target", ["int8", "int4"])
def test_quantize_integer_rounding_at_and_around_ties(qlib, oracle, dev, target):
    """The integer quantisers round x / scale without a division wherever the product with the reciprocal is provably
    far enough from k + 1/2; inputs built to sit exactly on, and a few ulps either side of, every tie k + 1/2 (and
    on the integers themselves) must still come out bit for bit as the oracle's divide-then-round."""
    q = qlib
    qmax = 127 if target == "int8" else 7
    rng = np.random.default_rng(17)
    for amax in (1.0, 3.1415927, 0.001953125, 1234.5677, 6.1e-5):
        scale = np.float32(np.float32(amax) / np.float32(qmax))
        k = np.arange(-qmax - 2, qmax + 2, dtype=np.float32)
        base = np.concatenate([(k + np.float32(0.5)) * scale, k * scale, (k + np.float32(0.4999)) * scale,
                               (k + np.float32(0.5001)) * scale]).astype(np.float32)
        vals = [base]
        for ulps in (1, 2, 3, 8, 64):
            up = base.copy()
            dn = base.copy()
            for _ in range(ulps):
                up = np.nextafter(up, np.float32(np.inf), dtype=np.float32)
                dn = np.nextafter(dn, np.float32(-np.inf), dtype=np.float32)
            vals += [up, dn]
        x = np.concatenate(vals + [rng.standard_normal(4096).astype(np.float32) * np.float32(amax / 3)])
        x = np.clip(x, -np.float32(amax), np.float32(amax)).astype(np.float32)
        x[0] = np.float32(amax)  # pins the matrix's amax, hence the scale
        if x.size % 16:
            x = np.concatenate([x, np.zeros(16 - x.size % 16, np.float32)])
        x = x.reshape(8, -1)  # an even number of columns (int4 packs pairs)
        xt = torch.from_numpy(x).to(dev)
        if target == "int8":
            got, s = q.quantize(xt, torch.int8)
            ref, s_ref = oracle.quantize_int8(x)
            assert np.array_equal(got.cpu().numpy(), ref), amax
        else:
            got, s = q.quantize_int4(xt)
            ref, s_ref = oracle.quantize_int4(x)
            assert np.array_equal(got.cpu().numpy(), ref), amax
        assert float(s) == s_ref
