"""Seeded random shapes through the library's own planning (no tuning): whatever kernel the planner picks -- lone CTA
with one or two K blocks per load, CTA pairs on 256 x 256 or 256 x 128 tiles, K slices inside one launch on clusters
of CTAs or CTA pairs, two-launch split-K, last-wave split -- the int8 accumulator must equal the oracle's bit for bit
and the scaled bf16 output must be within one ulp. Shapes are drawn so that every planning regime is hit (skinny,
few-tiles-long-K, mid-size, ragged edges) at sizes the CPU oracle finishes in well under a second each."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def _shapes(n, seed):
    rng = np.random.default_rng(seed)
    out = []
    regimes = [
        (lambda: (int(rng.integers(1, 70)), int(rng.integers(8, 7200)), 16 * int(rng.integers(1, 160)))),       # skinny
        (lambda: (int(rng.integers(1, 300)), int(rng.integers(8, 1300)), 16 * int(rng.integers(64, 1100)))),    # long K
        (lambda: (int(rng.integers(200, 1300)), int(rng.integers(200, 2100)), 16 * int(rng.integers(8, 600)))),  # mid-size
        (lambda: (int(rng.integers(1, 2100)), int(rng.integers(1, 2100)), 16 * int(rng.integers(1, 40)))),      # short K
    ]
    while len(out) < n:
        M, N, K = regimes[len(out) % len(regimes)]()
        if M * N * K <= 3_000_000_000:
            out.append((M, N, K))
    return out


@pytest.mark.parametrize("M,N,K", _shapes(48, 20240611))
def test_int8_default_plan_matches_oracle(qlib, oracle, dev, M, N, K):
    q = qlib
    ai = datagen.int8_uniform((M, K), seed=M * 7 + N, stream=0)
    bi = datagen.int8_uniform((N, K), seed=M * 7 + N, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    plan = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, None)
    acc = torch.full((M, N), -7, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True)
    ref = oracle.gemm_i8(ai, bi, True)
    assert np.array_equal(acc.cpu().numpy(), ref), plan
    sa, sb = datagen.scale_pair(M + K)
    c = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev), c, b_kmajor=True)
    bits = c.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(bits, oracle.scale_cast(ref, float(sa), float(sb), oracle.OUT_BF16)) <= 1, plan
    rc, st = q.device_status()
    assert rc == 0, (st, plan)


def test_the_random_shapes_cover_the_planning_regimes(qlib):
    """Host arithmetic only: the drawn shapes reach every kind of plan (so the test above exercises them)."""
    q = qlib
    kinds = set()
    for M, N, K in _shapes(48, 20240611):
        p = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, None)
        kinds.add((p["ctas_per_tile"], p["tile_n"], p["cluster_slices"] > 0, p["split_k"] > 1, p["k_blocks_per_load"]))
    assert any(k[0] == 2 and k[1] == 256 for k in kinds), kinds
    assert any(k[0] == 1 and k[2] for k in kinds), kinds          # lone-CTA cluster split
    assert any(k[0] == 1 and k[4] == 2 for k in kinds), kinds     # K-grouped loads
    assert any(k[0] == 1 and k[4] == 1 for k in kinds), kinds
