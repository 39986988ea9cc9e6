"""Parity of the CUDA GEMM path (through the C-ABI) with the CPU oracle, on seeded inputs.

Tiers:  int8  -> int32 accumulator bit-exact; scaled bf16 output within 1 bf16 ulp.
        fp8   -> max relative error (with an rms floor) <= 1e-2 against the fp32 oracle on the
                 dequantised inputs.
        fp16 / bf16 -> rel-L2 <= 1e-3 against fp32 accumulation.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3      # fp16 / bf16 tier
FP8_MAX_REL_TOL = 1e-2  # fp8 tier
BF16_ULP_TOL = 1       # int8 scaled-output tier


def _bits16(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _to_dev16(bits, dtype, dev):
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(dtype)


def _status_ok(q):
    rc, st = q.device_status()
    assert rc == 0, f"device status {st}"


SHAPES_16 = [
    (1, 1, 8), (1, 16, 8), (16, 8, 64), (128, 256, 64), (127, 255, 72), (129, 257, 136), (200, 300, 1000),
    (256, 512, 512), (300, 1000, 264), (512, 128, 2048), (1024, 1024, 1024),
]


@pytest.mark.parametrize("M,N,K", SHAPES_16)
@pytest.mark.parametrize("in_name", ["bf16", "fp16"])
def test_f16_kinds_fp32_out(qlib, oracle, dev, M, N, K, in_name):
    q = qlib
    a32 = datagen.normal((M, K), seed=M + N + K, stream=0)
    b32 = datagen.normal((N, K), seed=M + N + K, stream=1)
    rnd = oracle.round_bf16 if in_name == "bf16" else oracle.round_f16
    tdt = torch.bfloat16 if in_name == "bf16" else torch.float16
    a_bits, a_val = rnd(a32)
    b_bits, b_val = rnd(b32)
    a, b = _to_dev16(a_bits, tdt, dev), _to_dev16(b_bits, tdt, dev)
    c = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=True)
    ref = oracle.gemm_f32(a_val, b_val, True)
    got = c.cpu().numpy()
    assert np.isfinite(got).all()
    assert oracle.rel_l2(got, ref) <= REL_L2_TOL
    # tensor-core fp32 accumulation is far tighter than the tier: keep it honest
    assert oracle.rel_l2(got, oracle.gemm_f64(a_val, b_val, True)) <= 1e-5
    _status_ok(q)


def test_config1_fp16_1024_b_colmajor(qlib, oracle, dev):
    """FP16 GEMM M=N=K=1024, A row-major, B col-major [K,N] (= K-major), uniform[-1,1) seed 0, fp32 out."""
    q = qlib
    M = N = K = 1024
    a_bits, a_val = oracle.round_f16(datagen.uniform((M, K), seed=0, stream=0))
    b_bits, b_val = oracle.round_f16(datagen.uniform((N, K), seed=0, stream=1))
    a, b = _to_dev16(a_bits, torch.float16, dev), _to_dev16(b_bits, torch.float16, dev)
    c = torch.empty((M, N), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=True)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= REL_L2_TOL
    _status_ok(q)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 264, 136), (77, 130, 56), (512, 768, 320), (300, 1000, 264)])
@pytest.mark.parametrize("out_name", ["fp32", "bf16", "fp16"])
@pytest.mark.parametrize("relayout", [0, 1])
def test_bf16_row_major_b(qlib, oracle, dev, M, N, K, out_name, relayout):
    """B given as [K,N] row-major: read in place as an MN-major tensor-core operand when its rows are 16-byte
    aligned (relayout = 0), or relaid out to K-major by the transpose kernel first (relayout = 1, and always
    for an unaligned B such as N = 130)."""
    q = qlib
    tuning = q.Tuning(0, 0, 0, 0, 0, relayout)
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=7, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((K, N), seed=7, stream=1))
    a, b = _to_dev16(a_bits, torch.bfloat16, dev), _to_dev16(b_bits, torch.bfloat16, dev)
    odt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[out_name]
    c = torch.zeros((M, N), dtype=odt, device=dev)
    q.gemm(a, b, c, b_kmajor=False, tuning=tuning)
    ref = oracle.gemm_f32(a_val, b_val, False)
    got = c.float().cpu().numpy()
    tol = REL_L2_TOL if out_name == "fp32" else 4e-3  # one extra rounding to a 16-bit output
    assert oracle.rel_l2(got, ref) <= tol
    if out_name != "fp32":
        # The down-cast is one round-to-nearest-even of the fp32 accumulator: the 16-bit output equals
        # the rounding of the same kernel's fp32 output bit for bit (an ulp bound against the oracle's
        # differently ordered fp32 sum is meaningless where the sum cancels to near zero).
        c32 = torch.zeros((M, N), dtype=torch.float32, device=dev)
        q.gemm(a, b, c32, b_kmajor=False, tuning=tuning)
        kind = oracle.OUT_BF16 if out_name == "bf16" else oracle.OUT_F16
        assert np.array_equal(_bits16(c), oracle.scale_cast(c32.cpu().numpy(), 1.0, 1.0, kind))
    _status_ok(q)


@pytest.mark.parametrize("tile_n,pair", [(256, -1), (128, -1), (64, -1), (256, 1)])
def test_row_major_b_in_place_every_tile_shape(qlib, oracle, dev, tile_n, pair):
    """The in-place (MN-major) B path under every tile configuration, bf16, ragged N and K."""
    q = qlib
    M, N, K = 384, 1112, 456
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=13, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((K, N), seed=13, stream=1))
    a, b = _to_dev16(a_bits, torch.bfloat16, dev), _to_dev16(b_bits, torch.bfloat16, dev)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=False, tuning=q.Tuning(tile_n, 1, 0, 0, pair, 0))
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, False)) <= REL_L2_TOL
    _status_ok(q)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (300, 528, 400), (1024, 1024, 2048)])
@pytest.mark.parametrize("relayout", [0, 1])
def test_int8_and_fp8_row_major_b(qlib, oracle, dev, M, N, K, relayout):
    """8-bit operands with B [K,N] row-major: in place (128-column chunks) and through the relayout."""
    q = qlib
    tuning = q.Tuning(0, 0, 0, 0, 0, relayout)
    ai = datagen.int8_uniform((M, K), seed=K + 3, stream=0)
    bi = datagen.int8_uniform((K, N), seed=K + 3, stream=1)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.gemm(torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev), acc, b_kmajor=False, tuning=tuning)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, False))
    a32 = datagen.normal((M, K), seed=K, stream=0)
    b32 = datagen.normal((K, N), seed=K, stream=1)
    a_bits, a_val, sa = oracle.quantize_e4m3(a32)
    b_bits, b_val, sb = oracle.quantize_e4m3(b32)
    a = torch.from_numpy(a_bits).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b_bits).to(dev).view(torch.float8_e4m3fn)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c, b_kmajor=False, tuning=tuning)
    ref = oracle.gemm_f32(a_val, b_val, False) * (np.float32(sa) * np.float32(sb))
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= FP8_MAX_REL_TOL
    _status_ok(q)


def test_leading_dimensions_are_honoured(qlib, oracle, dev):
    """lda/ldb/ldc larger than the logical widths (the reference ignores ldA/ldB,
    src/include/gemm_utils.cuh:93,108); untouched padding must stay untouched."""
    q = qlib
    M, N, K = 150, 200, 96
    lda, ldb, ldc = 128, 104, 256
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=11, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=11, stream=1))
    A = torch.zeros((M, lda), dtype=torch.bfloat16, device=dev)
    B = torch.zeros((N, ldb), dtype=torch.bfloat16, device=dev)
    A[:, :K] = _to_dev16(a_bits, torch.bfloat16, dev)
    B[:, :K] = _to_dev16(b_bits, torch.bfloat16, dev)
    A[:, K:] = 1000.0  # poison: must never be read as part of the product
    B[:, K:] = 1000.0
    Cbuf = torch.full((M, ldc), -5.0, dtype=torch.float32, device=dev)
    q.gemm(A[:, :K], B[:, :K], Cbuf[:, :N], b_kmajor=True)
    got = Cbuf.cpu().numpy()
    assert oracle.rel_l2(got[:, :N], oracle.gemm_f32(a_val, b_val, True)) <= REL_L2_TOL
    assert np.all(got[:, N:] == -5.0)
    _status_ok(q)


INT8_SHAPES = [(1, 1, 16), (16, 32, 128), (128, 256, 128), (130, 260, 144), (257, 100, 1040), (512, 512, 4096),
               (1024, 1024, 1024)]


@pytest.mark.parametrize("M,N,K", INT8_SHAPES)
def test_int8_accumulator_bit_exact(qlib, oracle, dev, M, N, K):
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, True))
    _status_ok(q)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (130, 260, 144), (512, 512, 4096)])
@pytest.mark.parametrize("out_name", ["bf16", "fp16", "fp32"])
def test_int8_mixed_scaled_output(qlib, oracle, dev, M, N, K, out_name):
    """C = (A o Q_A) x (B o Q_B): scaled output within 1 bf16 ulp of cast(sA*sB*acc)."""
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=K + 1, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K + 1, stream=1)
    sa, sb = datagen.scale_pair(seed=K + 1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    odt = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[out_name]
    c = torch.zeros((M, N), dtype=odt, device=dev)
    q.int8_mm(a, b, tsa, tsb, c)
    acc = oracle.gemm_i8(ai, bi, True)
    if out_name == "bf16":
        ref_bits = oracle.scale_cast(acc, float(sa), float(sb), oracle.OUT_BF16)
        assert oracle.bf16_ulp_distance(_bits16(c), ref_bits) <= BF16_ULP_TOL
    elif out_name == "fp16":
        ref = oracle.f16_decode(oracle.scale_cast(acc, float(sa), float(sb), oracle.OUT_F16))
        assert np.allclose(c.float().cpu().numpy(), ref, rtol=2e-3, atol=1e-6)
    else:
        ref = oracle.scale_cast(acc, float(sa), float(sb), oracle.OUT_F32)
        assert np.allclose(c.cpu().numpy(), ref, rtol=1e-6, atol=0)
    _status_ok(q)


def _fp8_operands(oracle, dev, M, N, K, seed):
    a32 = datagen.normal((M, K), seed=seed, stream=0)
    b32 = datagen.normal((N, K), seed=seed, stream=1)
    a_bits, a_val, sa = oracle.quantize_e4m3(a32)
    b_bits, b_val, sb = oracle.quantize_e4m3(b32)
    a = torch.from_numpy(a_bits).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b_bits).to(dev).view(torch.float8_e4m3fn)
    return a, b, a_val, b_val, np.float32(sa), np.float32(sb)


@pytest.mark.parametrize("M", [16, 64, 256, 1024])
def test_fp8_sweep_shapes(qlib, oracle, dev, M):
    """FP8 e4m3, per-matrix scale amax/448, N=7168, K=2048, bf16 out (the skinny-to-square sweep;
    M=6144 is covered by the sampled test below)."""
    q = qlib
    N, K = 7168, 2048
    a, b, a_val, b_val, sa, sb = _fp8_operands(oracle, dev, M, N, K, seed=M)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.fp8_mm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c)
    ref = oracle.gemm_f32_blocked(a_val, b_val) * (sa * sb)
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= FP8_MAX_REL_TOL
    _status_ok(q)


@pytest.mark.parametrize("M,N,K", [(1, 16, 16), (100, 200, 300 // 16 * 16), (130, 270, 2064)])
@pytest.mark.parametrize("out_name", ["bf16", "fp32"])
def test_fp8_ragged(qlib, oracle, dev, M, N, K, out_name):
    q = qlib
    a, b, a_val, b_val, sa, sb = _fp8_operands(oracle, dev, M, N, K, seed=M * 3 + K)
    odt = {"fp32": torch.float32, "bf16": torch.bfloat16}[out_name]
    c = torch.zeros((M, N), dtype=odt, device=dev)
    q.fp8_mm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c)
    ref = oracle.gemm_f32(a_val, b_val, True) * (sa * sb)
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= FP8_MAX_REL_TOL
    _status_ok(q)


@pytest.mark.parametrize("tile_n,split_k", [(256, 2), (256, 4), (128, 2), (128, 3), (128, 8), (128, 16)])
def test_split_k_int8_stays_bit_exact(qlib, oracle, dev, tile_n, split_k):
    q = qlib
    M, N, K = 100, 520, 2048
    ai = datagen.int8_uniform((M, K), seed=5, stream=0)
    bi = datagen.int8_uniform((N, K), seed=5, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=q.Tuning(tile_n, split_k, 0, 0))
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, True))
    _status_ok(q)


@pytest.mark.parametrize("in_name", ["bf16", "fp8"])
@pytest.mark.parametrize("split_k", [2, 4, 7])
def test_split_k_floating(qlib, oracle, dev, in_name, split_k):
    q = qlib
    M, N, K = 64, 7168 // 8, 2048
    if in_name == "fp8":
        a, b, a_val, b_val, sa, sb = _fp8_operands(oracle, dev, M, N, K, seed=split_k)
        tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    else:
        a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=split_k, stream=0))
        b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=split_k, stream=1))
        a, b = _to_dev16(a_bits, torch.bfloat16, dev), _to_dev16(b_bits, torch.bfloat16, dev)
        sa = sb = np.float32(1.0)
        tsa = tsb = None
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, c, b_kmajor=True, tuning=q.Tuning(128, split_k, 0, 0))
    ref = oracle.gemm_f32(a_val, b_val, True) * (sa * sb)
    got = c.float().cpu().numpy()
    if in_name == "fp8":
        assert oracle.max_rel(got, ref) <= FP8_MAX_REL_TOL
    else:
        assert oracle.rel_l2(got, ref) <= 4e-3
    # split-K is a fixed-order two-pass sum: two runs give identical bits
    c2 = torch.zeros_like(c)
    q.mix_gemm(a, b, tsa, tsb, c2, b_kmajor=True, tuning=q.Tuning(128, split_k, 0, 0))
    assert torch.equal(c, c2)
    _status_ok(q)


@pytest.mark.parametrize("group_m,max_ctas", [(1, 0), (3, 0), (16, 5), (2, 1)])
def test_tile_order_and_persistence_do_not_change_results(qlib, oracle, dev, group_m, max_ctas):
    """Any grouping and any number of persistent CTAs (down to one CTA walking every tile)."""
    q = qlib
    M, N, K = 640, 1100, 192
    ai = datagen.int8_uniform((M, K), seed=9, stream=0)
    bi = datagen.int8_uniform((N, K), seed=9, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=q.Tuning(128, 1, group_m, max_ctas))
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, True))
    _status_ok(q)


def test_empty_and_degenerate_shapes(qlib, dev):
    q = qlib
    a = torch.zeros((0, 64), dtype=torch.bfloat16, device=dev)
    b = torch.zeros((32, 64), dtype=torch.bfloat16, device=dev)
    c = torch.zeros((0, 32), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=True)  # M = 0: nothing to do
    # K = 0: the empty sum is zero
    L = q.lib()
    cbuf = torch.full((4, 8), 3.0, dtype=torch.float32, device=dev)
    rc = L.qgemm_gemm(q.BF16, q.FP32, q.B_K_MAJOR, None, 0, None, 0, cbuf.data_ptr(), 8, 4, 8, 0, None)
    assert rc == q.OK
    torch.cuda.synchronize()
    assert torch.all(cbuf == 0)


def test_error_codes(qlib, dev):
    q = qlib
    L = q.lib()
    a = torch.zeros((128, 72), dtype=torch.bfloat16, device=dev)
    b = torch.zeros((128, 72), dtype=torch.bfloat16, device=dev)
    c = torch.zeros((128, 128), dtype=torch.float32, device=dev)
    # misaligned base pointer (2 bytes off) for a K-major operand
    rc = L.qgemm_gemm(q.BF16, q.FP32, q.B_K_MAJOR, a.data_ptr() + 2, 72, b.data_ptr(), 72, c.data_ptr(), 128, 128, 128,
                      64, None)
    assert rc == q.ERR_ALIGNMENT
    # leading dimension not a multiple of 16 bytes
    rc = L.qgemm_gemm(q.BF16, q.FP32, q.B_K_MAJOR, a.data_ptr(), 68, b.data_ptr(), 72, c.data_ptr(), 128, 128, 128, 64,
                      None)
    assert rc == q.ERR_ALIGNMENT
    # ld smaller than the row
    rc = L.qgemm_gemm(q.BF16, q.FP32, q.B_K_MAJOR, a.data_ptr(), 32, b.data_ptr(), 72, c.data_ptr(), 128, 128, 128, 64,
                      None)
    assert rc == q.ERR_INVALID_ARG
    # unsupported dtype pair
    rc = L.qgemm_gemm(q.BF16, q.INT32, q.B_K_MAJOR, a.data_ptr(), 72, b.data_ptr(), 72, c.data_ptr(), 128, 128, 128, 64,
                      None)
    assert rc == q.ERR_UNSUPPORTED
    rc = L.qgemm_gemm(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, a.data_ptr(), 72, b.data_ptr(), 72, c.data_ptr(), 128, 128, 128,
                      64, None)
    assert rc == q.ERR_UNSUPPORTED  # fp8 goes through qgemm_mix_gemm
    with pytest.raises(q.QgemmError):
        q.gemm(a.cpu(), b, c)


def test_unaligned_row_major_b_is_accepted(qlib, oracle, dev):
    """Row-major B is relaid out by the transpose kernel, which takes any alignment (N odd here)."""
    q = qlib
    M, N, K = 64, 75, 96
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=21, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((K, N), seed=21, stream=1))
    a, b = _to_dev16(a_bits, torch.bfloat16, dev), _to_dev16(b_bits, torch.bfloat16, dev)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.gemm(a, b, c, b_kmajor=False)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, False)) <= REL_L2_TOL


def test_linearity_at_full_size_int8(qlib, oracle, dev):
    """Size-independent property at the full 8192^3 int8 configuration: the product is linear in A,
    so (A1 + A2) x B == A1 x B + A2 x B exactly in int32, and sampled row bands match the oracle."""
    q = qlib
    M = N = K = 8192
    a1 = datagen.int8_uniform((M, K), seed=31, stream=0) // 2
    a2 = datagen.int8_uniform((M, K), seed=31, stream=2) // 2
    bi = datagen.int8_uniform((N, K), seed=31, stream=1)
    b = torch.from_numpy(bi).to(dev)
    outs = []
    for ai in (a1, a2, (a1 + a2).astype(np.int8)):
        acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
        q.gemm(torch.from_numpy(ai).to(dev), b, acc, b_kmajor=True)
        outs.append(acc)
    assert torch.equal(outs[0] + outs[1], outs[2])
    got = outs[2].cpu().numpy()
    asum = (a1 + a2).astype(np.int8)
    for m0 in (0, 4088, 8184):  # first, middle (straddling a tile edge) and last rows
        assert np.array_equal(got[m0:m0 + 8], oracle.gemm_i8_rows(asum, bi, m0, m0 + 8))
    _status_ok(q)


def test_output_larger_than_4_gib_uses_64_bit_addressing(qlib, oracle, dev):
    """M x N x sizeof(C) beyond 2^32 bytes: row offsets must be computed in 64 bits on every store path."""
    q = qlib
    M, N, K = 70000, 32768, 64
    ai = datagen.int8_uniform((M, K), seed=77, stream=0)
    bi = datagen.int8_uniform((N, K), seed=77, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    one = torch.ones(1, device=dev)
    c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)  # 4.6 GB
    assert c.numel() * 2 > 2 ** 32
    for tuning in (None, q.Tuning(128, 1, 0, 0, -1, 0)):  # CTA pairs, and the lone-CTA kernel
        c.fill_(-7.0)
        q.mix_gemm(a, b, one, one, c, b_kmajor=True, tuning=tuning)
        for m0 in (0, 32767, 65530, M - 5):
            got = c[m0:m0 + 5].float().cpu().numpy()
            ref = oracle.gemm_i8_rows(ai, bi, m0, m0 + 5).astype(np.float32)
            ref_bits = oracle.round_bf16(ref)[0]
            assert np.array_equal(c[m0:m0 + 5].view(torch.int16).cpu().numpy().view(np.uint16), ref_bits), m0
            assert np.isfinite(got).all()
    del c
    torch.cuda.empty_cache()
    _status_ok(q)


def test_config2_bf16_8192_row_major_b_sampled(qlib, oracle, dev):
    """BF16 8192^3, A and B row-major, bf16 out: sampled row bands against the oracle (rel-L2)."""
    q = qlib
    M = N = K = 8192
    a32 = datagen.normal((M, K), seed=2, stream=0)
    b32 = datagen.normal((K, N), seed=2, stream=1)
    a = torch.from_numpy(a32).to(dev).to(torch.bfloat16)
    b = torch.from_numpy(b32).to(dev).to(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.gemm(a, b, c, b_kmajor=False)
    _, b_val = oracle.round_bf16(b32)
    bt = np.ascontiguousarray(b_val.T)
    got = c.float().cpu().numpy()
    for m0 in (0, 4090, 8180):
        _, a_val = oracle.round_bf16(a32[m0:m0 + 12])
        ref = oracle.gemm_f32_blocked(a_val, bt)
        assert oracle.rel_l2(got[m0:m0 + 12], ref) <= 4e-3  # bf16 output rounding on top of the 1e-3 tier
    _status_ok(q)


def test_fp8_6144_sampled(qlib, oracle, dev):
    q = qlib
    M, N, K = 6144, 7168, 2048
    a, b, a_val, b_val, sa, sb = _fp8_operands(oracle, dev, M, N, K, seed=6144)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.fp8_mm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c)
    got = c.float().cpu().numpy()
    for m0 in (0, 3000, 6100):
        ref = oracle.gemm_f32_blocked(a_val[m0:m0 + 44], b_val) * (sa * sb)
        assert oracle.max_rel(got[m0:m0 + 44], ref) <= FP8_MAX_REL_TOL
    _status_ok(q)


def test_cpp_templates_are_exported_for_the_reference_harness(qlib):
    """The Itanium-mangled specialisations an unmodified tests/cuda_benchmark.cpp links against."""
    L = C.CDLL(qlib.LIB_PATH)
    for sym in ("_Z14GEMM_kernel_v1I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
                "_Z14GEMM_kernel_v2I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
                "_Z14GEMM_kernel_v3I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
                "_Z16GEMM_kernel_v3_1I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm",
                "_Z14GEMM_kernel_v4I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm"):
        getattr(L, sym)


def test_cpp_template_entry_runs(qlib, oracle, dev):
    """Call GEMM_kernel_v3<bf16,float> exactly as the reference harness does (row-major B, default stream)."""
    L = C.CDLL(qlib.LIB_PATH)
    fn = getattr(L, "_Z14GEMM_kernel_v3I13__nv_bfloat16fEvPKT_mS3_mPT0_mmmm")
    fn.restype = None
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                   C.c_size_t]
    M, N, K = 512, 384, 256
    af = oracle.harness_fill(M * K, False).reshape(M, K)
    bf = oracle.harness_fill(K * N, True).reshape(K, N)
    a_bits, a_val = oracle.round_bf16(af)
    b_bits, b_val = oracle.round_bf16(bf)
    a, b = _to_dev16(a_bits, torch.bfloat16, dev), _to_dev16(b_bits, torch.bfloat16, dev)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    fn(a.data_ptr(), K, b.data_ptr(), N, c.data_ptr(), N, M, N, K)
    torch.cuda.synchronize()
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, False)) <= REL_L2_TOL
