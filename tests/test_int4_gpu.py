"""Int4 (the roadmap precision the reference names but never implements, develop.md:9-12): packed signed 4-bit
operands, two per byte. The GEMM is exact (int32 sums) against the CPU oracle, the scaled 16-bit output within one
ulp, and the quantiser bit-exact."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def _pack(v):
    v = v.astype(np.int8)
    return ((v[:, 0::2] & 0xf) | ((v[:, 1::2] & 0xf) << 4)).astype(np.uint8)


def _rand_int4(shape, seed, stream):
    return (datagen.int8_uniform(shape, seed=seed, stream=stream).astype(np.int16) % 16 - 8).astype(np.int8)


@pytest.mark.parametrize("M,N,K", [(1, 8, 2), (16, 24, 32), (130, 270, 250), (256, 512, 1024), (300, 1000, 4096),
                                    (1024, 1024, 2048)])
def test_int4_gemm_exact(qlib, oracle, dev, M, N, K):
    q = qlib
    a = _rand_int4((M, K), seed=K, stream=0)
    b = _rand_int4((N, K), seed=K, stream=1)
    ap, bp = _pack(a), _pack(b)
    assert np.array_equal(oracle.unpack_int4(ap), a)
    at, bt = torch.from_numpy(ap).to(dev), torch.from_numpy(bp).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    q.int4_mm(at, bt, None, None, acc)
    want = oracle.gemm_i4(ap, bp)
    assert np.array_equal(acc.cpu().numpy(), want)
    assert np.array_equal(want, oracle.gemm_i8(a, b, True))
    # scaled bf16 output
    sa, sb = torch.tensor([0.11], device=dev), torch.tensor([0.07], device=dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.int4_mm(at, bt, sa, sb, c)
    ref_bits = oracle.scale_cast(want, float(sa.item()), float(sb.item()), oracle.OUT_BF16)
    got_bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(got_bits, ref_bits) <= 1
    rc, st = q.device_status()
    assert rc == 0, st


def test_int4_strided_operands_and_errors(qlib, oracle, dev):
    q = qlib
    M, N, K = 64, 96, 128
    a = _rand_int4((M, K), seed=3, stream=0)
    b = _rand_int4((N, K), seed=3, stream=1)
    big_a = torch.zeros((M, K // 2 + 8), dtype=torch.uint8, device=dev)
    big_a[:, :K // 2] = torch.from_numpy(_pack(a)).to(dev)
    big_a[:, K // 2:] = 0x77  # must never be read as part of the product
    bt = torch.from_numpy(_pack(b)).to(dev)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.int4_mm(big_a[:, :K // 2], bt, None, None, acc)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(a, b, True))
    # a row-major [K, N] B cannot be packed along K: rejected
    rc = q.lib().qgemm_gemm_ex(q.INT4, q.INT32, q.B_ROW_MAJOR, big_a.data_ptr(), K, bt.data_ptr(), N, None, None,
                               acc.data_ptr(), N, M, N, K, None, None)
    assert rc == q.ERR_UNSUPPORTED
    # an odd K or leading dimension
    rc = q.lib().qgemm_gemm_ex(q.INT4, q.INT32, q.B_K_MAJOR, big_a.data_ptr(), K, bt.data_ptr(), K, None, None,
                               acc.data_ptr(), N, M, N, K - 1, None, None)
    assert rc == q.ERR_INVALID_ARG
    assert q.workspace_query(q.INT4, q.B_K_MAJOR, M, N, K) >= (M + N) * K


@pytest.mark.parametrize("shape", [(1, 2), (33, 70), (256, 1024), (1000, 514)])
@pytest.mark.parametrize("in_dtype", [torch.float32, torch.bfloat16])
def test_quantize_int4_bit_exact(qlib, oracle, dev, shape, in_dtype):
    q = qlib
    x32 = datagen.normal(shape, seed=shape[1], stream=0)
    if in_dtype == torch.bfloat16:
        bits, x32 = oracle.round_bf16(x32)
        x = torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)
    else:
        x = torch.from_numpy(x32).to(dev)
    packed, scale = q.quantize_int4(x)
    want, want_scale = oracle.quantize_int4(x32)
    assert np.float32(scale.item()) == np.float32(want_scale)
    assert np.array_equal(packed.cpu().numpy(), want)
    # and the round trip through the GEMM: (x/s) x (x/s)^T with the two scales restores x x^T to int4 accuracy
    if shape[0] >= 33:
        c = torch.zeros((shape[0], shape[0]), dtype=torch.float32, device=dev)
        q.int4_mm(packed, packed, scale, scale, c)
        deq = oracle.unpack_int4(want).astype(np.float32) * np.float32(want_scale)
        ref = oracle.gemm_f32(deq, deq, True)
        assert oracle.rel_l2(c.cpu().numpy(), ref) <= 1e-5


def test_quantize_int4_all_zero_and_odd_columns(qlib, dev):
    q = qlib
    z = torch.zeros((4, 8), dtype=torch.float32, device=dev)
    packed, scale = q.quantize_int4(z)
    assert float(scale.item()) == 1.0 and bool((packed == 0).all())
    with pytest.raises(q.QgemmError):
        q.quantize_int4(torch.zeros((4, 7), dtype=torch.float32, device=dev))
