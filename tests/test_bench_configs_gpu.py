"""The benchmarked configurations, at full size and along the code path the benchmark times, against the CPU oracle.

Each case builds the operands the way bench.py does, runs the product through the C-ABI with the same tuning the
timed loop uses, and compares sampled row bands (first rows, rows straddling a tile edge, last rows) with the
oracle (oracle/sampled.py); tolerances are the tiers' and are written there:

  * BF16 8192^3, A and B row-major, B relaid out by the transpose kernel (relayout_b = 1), bf16 out;
    and the 512 x 256 wide-pair kernel on a K-major B, forced and by the library's own choice
  * int8 8192^3 with per-matrix scales: the SCALED bf16 output (<= 1 bf16 ulp), not only the int32 accumulator
  * the column-sharded int8 32768 x 32768 x 8192: one rank's shape (32768 x N/g x 8192 for g = 2, 4, 8) for the two
    ranks either side of a rank boundary, checked on the columns next to that boundary against the oracle run on
    the GLOBAL B, int32 bit-exact and bf16 within 1 ulp
  * block-scaled FP8 4096 x 7168 x 7168 (row-band form of the block-scaled oracle)
  * bf16_mm(a, b, as, bs, c) (src/gemm/sm80_gemm_kernel.cu:4-12)
"""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen, sharding

pytestmark = pytest.mark.gpu


def _status_ok(q):
    rc, st = q.device_status()
    assert rc == 0, f"device status {st}"


def _bits16(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.fixture(scope="module")
def sampled(oracle):
    from oracle import sampled as s
    return s


@pytest.fixture(scope="module")
def bf16_8192(oracle, dev):
    """The BF16 configuration's operands (seed 2, as bench.py): A [M,K] and B [K,N] row-major on the device, and
    the exact fp32 values of A's rows and of B^T for the oracle."""
    M = N = K = 8192
    a_h = torch.from_numpy(datagen.normal((M, K), 2, 0)).to(torch.bfloat16)
    b_h = torch.from_numpy(datagen.normal((K, N), 2, 1)).to(torch.bfloat16)
    bt_val = np.ascontiguousarray(b_h.float().numpy().T)
    return dict(M=M, N=N, K=K, a_h=a_h, a=a_h.to(dev), b=b_h.to(dev), bt_val=bt_val)


def test_config2_relayout_path_as_benchmarked(qlib, sampled, dev, bf16_8192):
    """relayout_b = 1: transpose kernel -> K-major scratch -> wide-pair kernel, bf16 out: the step bench.py times."""
    q, w = qlib, bf16_8192
    tuning = q.Tuning(0, 0, 0, 0, 0, 1)
    c = torch.zeros((w["M"], w["N"]), dtype=torch.bfloat16, device=dev)
    q.gemm(w["a"], w["b"], c, b_kmajor=False, tuning=tuning)
    res = sampled.check_float(lambda m0, m1: w["a_h"][m0:m1].float().numpy(), w["bt_val"],
                              lambda m0, m1: c[m0:m1].float().cpu().numpy(), w["M"], "f16", out_16bit=True)
    assert res["ok"], res
    # the library default (B read in place as an MN-major operand), which bench.py times beside it as `direct_b`
    c2 = torch.zeros_like(c)
    q.gemm(w["a"], w["b"], c2, b_kmajor=False)
    res = sampled.check_float(lambda m0, m1: w["a_h"][m0:m1].float().numpy(), w["bt_val"],
                              lambda m0, m1: c2[m0:m1].float().cpu().numpy(), w["M"], "f16", out_16bit=True)
    assert res["ok"], res
    _status_ok(q)


@pytest.mark.parametrize("forced", [True, False])
def test_config2_wide_pair_kernel_kmajor_b(qlib, sampled, dev, bf16_8192, forced):
    q, w = qlib, bf16_8192
    bt = q.transpose(w["b"])  # [N,K] K-major
    tuning = q.Tuning(0, 0, 0, 0, 2, 0) if forced else None
    plan = q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, w["M"], w["N"], w["K"], tuning)
    assert plan["tile_m"] == 512 and plan["ctas_per_tile"] == 2, plan  # the kernel the headline number is taken on
    c = torch.zeros((w["M"], w["N"]), dtype=torch.bfloat16, device=dev)
    q.gemm(w["a"], bt, c, b_kmajor=True, tuning=tuning)
    res = sampled.check_float(lambda m0, m1: w["a_h"][m0:m1].float().numpy(), w["bt_val"],
                              lambda m0, m1: c[m0:m1].float().cpu().numpy(), w["M"], "f16", out_16bit=True)
    assert res["ok"], res
    _status_ok(q)


def test_config3_int8_8192_scaled_bf16_output(qlib, sampled, dev):
    q = qlib
    M = N = K = 8192
    ai = datagen.int8_uniform((M, K), 2, 0)
    bi = datagen.int8_uniform((N, K), 2, 1)
    sa, sb = datagen.scale_pair(2)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.int8_mm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c)
    res = sampled.check_int8(ai, bi, lambda m0, m1: _bits16(c[m0:m1]), "bf16", sa, sb)
    assert res["ok"], res
    _status_ok(q)


@pytest.fixture(scope="module")
def sharded_int8(dev):
    """Global operands of the sharded configuration: A [32768, 8192] replicated, B [32768, 8192] K-major."""
    M, N, K = 32768, 32768, 8192
    ai = datagen.int8_uniform((M, K), 2, 0)
    bi = datagen.int8_uniform((N, K), 2, 1)
    return dict(M=M, N=N, K=K, ai=ai, bi=bi, a=torch.from_numpy(ai).to(dev))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_config5_rank_shapes_across_a_rank_boundary(qlib, sampled, dev, sharded_int8, world):
    """Ranks world/2 - 1 and world/2 meet at global column 16384, a rank boundary of the 2-, 4- and 8-way split
    alike. Each runs its own M x N/world x K product on its slice of B; the columns either side of the boundary
    (and of the slice's other edge) are compared with the oracle on the global B."""
    q, w = qlib, sharded_int8
    sa, sb = datagen.scale_pair(2)
    tsa, tsb = torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)
    for rank in (world // 2 - 1, world // 2):
        n0, n1 = sharding.partition_columns(w["N"], world, rank)
        assert n1 - n0 == w["N"] // world
        b_slice = torch.from_numpy(w["bi"][n0:n1]).to(dev)
        width = n1 - n0
        windows = [(0, 64), (width - 64, width)]
        c = torch.zeros((w["M"], width), dtype=torch.bfloat16, device=dev)
        sharding.sharded_mix_gemm(w["a"], b_slice, tsa, tsb, c)
        res = sampled.check_int8(w["ai"], w["bi"][n0:n1], lambda m0, m1: _bits16(c[m0:m1]), "bf16", sa, sb,
                                 cols=windows)
        assert res["ok"], (world, rank, res)
        del c
        if world == 8:  # the accumulator itself, bit for bit
            acc = torch.zeros((w["M"], width), dtype=torch.int32, device=dev)
            q.gemm(w["a"], b_slice, acc, b_kmajor=True)
            res = sampled.check_int8(w["ai"], w["bi"][n0:n1], lambda m0, m1: acc[m0:m1].cpu().numpy(), "int32",
                                     cols=windows)
            assert res["ok"], (world, rank, res)
            del acc
        torch.cuda.empty_cache()
    _status_ok(q)


def test_block_scaled_fp8_at_the_benchmarked_shape(qlib, oracle, sampled, dev):
    q = qlib
    M, N, K = 4096, 7168, 7168
    a32 = torch.from_numpy(datagen.normal((M, K), 2, 0))
    b32 = torch.from_numpy(datagen.normal((N, K), 2, 1))
    s0, s1 = a32.abs().max() / 448.0, b32.abs().max() / 448.0
    a_h, b_h = (a32 / s0).to(torch.float8_e4m3fn), (b32 / s1).to(torch.float8_e4m3fn)
    kbs, nbs = K // 128, N // 128
    rng = np.random.default_rng(7)
    a_scale = ((rng.random((kbs, M), dtype=np.float32) * 0.5 + 0.75) * float(s0)).astype(np.float32)
    b_scale = ((rng.random((kbs, nbs), dtype=np.float32) * 0.5 + 0.75) * float(s1)).astype(np.float32)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.fp8_block_mm(a_h.to(dev), b_h.to(dev), torch.from_numpy(a_scale).to(dev), torch.from_numpy(b_scale).to(dev), c,
                   reference_layout=False)
    a_bits = a_h.view(torch.uint8).numpy()
    bt_val = oracle.e4m3_decode(b_h.view(torch.uint8).numpy())
    res = sampled.check_block_scaled(lambda m0, m1: oracle.e4m3_decode(a_bits[m0:m1]), bt_val, a_scale, b_scale,
                                     lambda m0, m1: c[m0:m1].float().cpu().numpy(), M)
    assert res["ok"], res
    _status_ok(q)


@pytest.mark.parametrize("scaled", [False, True])
def test_bf16_mm_entry_point(qlib, oracle, dev, scaled):
    """bf16_mm(a, b, as, bs, c): a [m,k], b [n,k] (n = b.size(0)), optional per-matrix scales, c [m,n]."""
    q = qlib
    M, N, K = 300, 520, 1032
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), 11, 0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), 11, 1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    sa, sb = (np.float32(0.5), np.float32(3.0)) if scaled else (np.float32(1), np.float32(1))
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    q.bf16_mm(a, b, torch.tensor([sa], device=dev) if scaled else None,
              torch.tensor([sb], device=dev) if scaled else None, c)
    ref = oracle.gemm_f32(a_val, b_val, True) * (sa * sb)
    assert oracle.rel_l2(c.cpu().numpy(), ref) <= 1e-3
    _status_ok(q)
