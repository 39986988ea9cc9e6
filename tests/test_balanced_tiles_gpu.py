"""Balanced column tiling (opt-in, QGEMM_BALANCE=1): a problem with fewer equal tiles than SMs (small M) has the
sixteen-column units of N dealt out over as many tile columns as there are SMs, tile widths differing by at most 16.
Same sums as the equal tiling (each output element is one CTA's K loop in the same order), so the two must agree bit
for bit; and with the switch on, the skinny FP8 shapes of the sweep (M = 16, 64, 256 at N = 7168, K = 2048) must be
planned that way. The switch is read from the environment when the library is loaded: the tests set it and have the
library read its environment again."""
import os

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def balanced_on(qlib):
    os.environ["QGEMM_BALANCE"] = "1"
    qlib.lib().qgemm_reload_env()
    yield
    del os.environ["QGEMM_BALANCE"]
    qlib.lib().qgemm_reload_env()
    assert qlib.plan_query(qlib.FP8_E4M3, qlib.BF16, qlib.B_K_MAJOR, 16, 7168, 2048, None)["balanced_tiles"] == 0


@pytest.mark.parametrize("M", [16, 64, 256])
def test_skinny_fp8_shapes_are_planned_balanced(qlib, M):
    q = qlib
    plan = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, M, 7168, 2048, None)
    m_tiles = -(-M // 128)
    assert plan["balanced_tiles"] * m_tiles == 148 == plan["ctas"], plan
    assert plan["split_k"] == 1 and plan["ctas_per_tile"] == 1
    # 448 units over 148 (74) tile columns: 48- and 64-wide (96- and 112-wide) tiles
    assert plan["min_tile_n"] == (48 if M <= 128 else 96), plan


@pytest.mark.parametrize("M,N,K", [(16, 7168, 2048), (64, 7168, 2048), (256, 7168, 2048), (100, 7000, 528),
                                    (130, 1000, 272), (1, 40, 16), (33, 48, 4096), (128, 2360, 1024)])
def test_balanced_equals_equal_tiles_int8_exact(qlib, oracle, dev, M, N, K):
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=M + N, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M + N, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    bal = torch.full((M, N), -5, dtype=torch.int32, device=dev)
    q.gemm(a, b, bal, b_kmajor=True)
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, None)
    eq = torch.full((M, N), -6, dtype=torch.int32, device=dev)
    q.gemm(a, b, eq, b_kmajor=True, tuning=q.Tuning(plan["tile_n"], 1, 0, 0, -1, 0))  # explicit tile width: equal tiles
    assert torch.equal(bal, eq)
    assert np.array_equal(bal.cpu().numpy(), oracle.gemm_i8(ai, bi, True))
    rc, st = q.device_status()
    assert rc == 0, st


@pytest.mark.parametrize("out_name", ["bf16", "fp32"])
@pytest.mark.parametrize("M,N,K", [(16, 7168, 2048), (256, 7168, 2048), (48, 1000, 1040)])
def test_balanced_fp8_scaled_output(qlib, oracle, dev, M, N, K, out_name):
    """fp8 tier through the balanced tiles, including an output whose rows are not 16-byte multiples (N = 1000 with
    a view offset is covered by the element path: ldc = N + 3)."""
    q = qlib
    a_bits, a_val, sa = oracle.quantize_e4m3(datagen.normal((M, K), seed=K + M, stream=0))
    b_bits, b_val, sb = oracle.quantize_e4m3(datagen.normal((N, K), seed=K + M, stream=1))
    a = torch.from_numpy(a_bits).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b_bits).to(dev).view(torch.float8_e4m3fn)
    odt = {"bf16": torch.bfloat16, "fp32": torch.float32}[out_name]
    ldc = N + 3 if N == 1000 else N
    buf = torch.zeros((M, ldc), dtype=odt, device=dev)
    c = buf[:, :N]
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, M, N, K, None)["balanced_tiles"] > 0
    q.fp8_mm(a, b, torch.tensor([np.float32(sa)], device=dev), torch.tensor([np.float32(sb)], device=dev), c)
    ref = oracle.gemm_f32_blocked(a_val, b_val) * (np.float32(sa) * np.float32(sb))
    assert oracle.max_rel(c.float().cpu().numpy(), ref) <= 1e-2
    if ldc != N:
        assert float(buf[:, N:].abs().max()) == 0.0  # nothing written past the row's end
    rc, st = q.device_status()
    assert rc == 0, st
