"""The sampled checker (oracle/sampled.py) that the full-size GPU tests and bench.py's `oracle_check` rely on, exercised
on the CPU: a result produced by the oracle itself passes every tier, and a result with one corrupted element in a
sampled band fails -- the checker can tell right from wrong before it is trusted with a GPU result."""
import numpy as np
import pytest

from qgemm_b200 import datagen


@pytest.fixture(scope="module")
def sampled(oracle):
    from oracle import sampled as s
    return s


def test_row_bands_cover_first_middle_tile_edge_and_last(sampled):
    starts, rows = sampled.row_bands(8192, 12)
    assert rows == 12 and starts[0] == 0 and starts[-1] == 8192 - 12
    assert any(s < 4096 <= s + rows for s in starts)  # a band straddling the tile edge at row 4096
    starts, rows = sampled.row_bands(5, 12)
    assert rows == 5 and starts == [0]


def test_int8_tiers_accept_the_oracle_and_reject_a_flipped_element(oracle, sampled):
    M, N, K = 600, 200, 256
    a = datagen.int8_uniform((M, K), 5, 0)
    bt = datagen.int8_uniform((N, K), 5, 1)
    acc = oracle.gemm_i8(a, bt, True)
    assert sampled.check_int8(a, bt, lambda m0, m1: acc[m0:m1], "int32")["ok"]
    bad = acc.copy()
    bad[M - 1, 17] += 1
    assert not sampled.check_int8(a, bt, lambda m0, m1: bad[m0:m1], "int32")["ok"]
    sa, sb = 0.004, 0.007
    bits = oracle.scale_cast(acc, sa, sb, oracle.OUT_BF16)
    res = sampled.check_int8(a, bt, lambda m0, m1: bits[m0:m1], "bf16", sa, sb, cols=[(0, 64), (N - 64, N)])
    assert res["ok"] and res["max_bf16_ulp"] == 0
    off = bits.copy()
    off[0, 3] += 2  # two units in the last place
    assert not sampled.check_int8(a, bt, lambda m0, m1: off[m0:m1], "bf16", sa, sb, cols=[(0, 64)])["ok"]


def test_float_and_block_scaled_tiers(oracle, sampled):
    M, N, K = 300, 256, 384
    _, a_val = oracle.round_bf16(datagen.normal((M, K), 6, 0))
    _, bt_val = oracle.round_bf16(datagen.normal((N, K), 6, 1))
    ref = oracle.gemm_f32(a_val, bt_val, True)
    ok = sampled.check_float(lambda m0, m1: a_val[m0:m1], bt_val, lambda m0, m1: ref[m0:m1], M, "f16", out_16bit=False)
    assert ok["ok"] and ok["worst"] < 1e-5
    wrong = ref.copy()
    wrong[:12] *= 1.01
    assert not sampled.check_float(lambda m0, m1: a_val[m0:m1], bt_val, lambda m0, m1: wrong[m0:m1], M, "f16",
                                   out_16bit=False)["ok"]
    kbs, nbs = K // 128, N // 128
    rng = np.random.default_rng(1)
    a_scale = (rng.random((kbs, M), dtype=np.float32) + 0.5).astype(np.float32)
    b_scale = (rng.random((kbs, nbs), dtype=np.float32) + 0.5).astype(np.float32)
    full = oracle.gemm_fp8_block_scaled(a_val, bt_val, a_scale, b_scale)
    res = sampled.check_block_scaled(lambda m0, m1: a_val[m0:m1], bt_val, a_scale, b_scale, lambda m0, m1: full[m0:m1], M)
    assert res["ok"] and res["worst"] == 0.0  # the row-band form of the oracle equals the whole-matrix form
