"""Block-scaled FP8 GEMM (the reference's fp8_mm semantics, src/mix_gemm/hip_mix_gemm_kernel.cpp:249-378)
through the C-ABI against the CPU oracle. Tolerance: the FP8 tier, max relative error <= 1e-2 with the
denominator floored at 1e-2 * rms(ref); in practice the only differences are fp32 summation order and the
final rounding to bf16."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

FP8_MAX_REL_TOL = 1e-2


def _case(oracle, dev, M, N, K, seed):
    a32 = datagen.normal((M, K), seed=seed, stream=0)
    b32 = datagen.normal((N, K), seed=seed, stream=1)
    kbs, nbs = -(-K // 128), -(-N // 128)
    # per-block quantisation: every block gets its own amax/448 scale, as a block-scaled producer would emit
    a_scale = np.empty((kbs, M), np.float32)
    b_scale = np.empty((kbs, nbs), np.float32)
    a_q = np.empty((M, K), np.float32)
    b_q = np.empty((N, K), np.float32)
    for kb in range(kbs):
        ks = slice(kb * 128, min(K, kb * 128 + 128))
        am = np.maximum(np.abs(a32[:, ks]).max(axis=1), 1e-8)
        a_scale[kb] = am / 448.0
        a_q[:, ks] = a32[:, ks] / a_scale[kb][:, None]
        for nb in range(nbs):
            ns = slice(nb * 128, min(N, nb * 128 + 128))
            bm = max(float(np.abs(b32[ns, ks]).max()), 1e-8)
            b_scale[kb, nb] = bm / 448.0
            b_q[ns, ks] = b32[ns, ks] / b_scale[kb, nb]
    a_bits = torch.from_numpy(a_q).to(torch.float8_e4m3fn)
    b_bits = torch.from_numpy(b_q).to(torch.float8_e4m3fn)
    a_val = oracle.e4m3_decode(a_bits.view(torch.uint8).numpy())
    b_val = oracle.e4m3_decode(b_bits.view(torch.uint8).numpy())
    return a_bits.to(dev), b_bits.to(dev), a_val, b_val, a_scale, b_scale


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 256, 512), (100, 200, 384), (300, 520, 1040),
                                    (1, 16, 16), (512, 7168 // 4, 2048)])
@pytest.mark.parametrize("reference_layout", [True, False])
def test_block_scaled_fp8_matches_oracle(qlib, oracle, dev, M, N, K, reference_layout):
    q = qlib
    a, b, a_val, b_val, a_scale, b_scale = _case(oracle, dev, M, N, K, seed=M + K)
    tas, tbs = torch.from_numpy(a_scale).to(dev), torch.from_numpy(b_scale).to(dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    if reference_layout:  # a: [m,k] col-major = contiguous [k,m]; b: [k,n] row-major
        q.fp8_block_mm(a.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn),
                       b.view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), tas, tbs, c, True)
    else:
        q.fp8_block_mm(a, b, tas, tbs, c, False)
    ref = oracle.gemm_fp8_block_scaled(a_val, b_val, a_scale, b_scale)
    got = c.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert oracle.max_rel(got, ref) <= FP8_MAX_REL_TOL
    assert oracle.rel_l2(got, ref) <= 4e-3  # bf16 output rounding
    rc, st = q.device_status()
    assert rc == 0, st


def test_block_scaled_fp32_out_and_unit_scales_equal_plain_gemm(qlib, oracle, dev):
    """With all scales 1 the block-scaled product is the plain FP8 product (up to fp32 summation order)."""
    q = qlib
    M, N, K = 256, 384, 1024
    a = torch.randn((M, K), device=dev).to(torch.float8_e4m3fn)
    b = torch.randn((N, K), device=dev).to(torch.float8_e4m3fn)
    ones_a = torch.ones((K // 128, M), dtype=torch.float32, device=dev)
    ones_b = torch.ones((K // 128, N // 128), dtype=torch.float32, device=dev)
    c_bs = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.fp8_block_mm(a, b, ones_a, ones_b, c_bs, False)
    c_plain = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.mix_gemm(a, b, None, None, c_plain, b_kmajor=True)
    assert oracle.rel_l2(c_bs.cpu().numpy(), c_plain.cpu().numpy()) <= 1e-6


def test_block_scaled_unaligned_output_and_errors(qlib, oracle, dev):
    q = qlib
    M, N, K = 130, 77, 256  # ldc * 2 bytes is not a multiple of 16: element-store path
    a, b, a_val, b_val, a_scale, b_scale = _case(oracle, dev, M, N, K, seed=9)
    tas, tbs = torch.from_numpy(a_scale).to(dev), torch.from_numpy(b_scale).to(dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.fp8_block_mm(a, b, tas, tbs, c, False)
    ref = oracle.gemm_fp8_block_scaled(a_val, b_val, a_scale, b_scale)
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= FP8_MAX_REL_TOL
    L = q.lib()
    rc = L.qgemm_fp8_block_scaled_gemm(q.INT32, 0, 1, a.data_ptr(), K, b.data_ptr(), K, tas.data_ptr(), tbs.data_ptr(),
                                       c.data_ptr(), N, M, N, K, None)
    assert rc == q.ERR_UNSUPPORTED
    rc = L.qgemm_fp8_block_scaled_gemm(q.BF16, 0, 1, a.data_ptr(), K, b.data_ptr(), K, None, tbs.data_ptr(),
                                       c.data_ptr(), N, M, N, K, None)
    assert rc == q.ERR_INVALID_ARG
