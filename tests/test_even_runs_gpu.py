"""The K range of all tiles dealt out evenly over the CTA pairs (GemmParams::sk_parts): the K blocks of the 256 x 256 tiles,
laid end to end in tile order, are cut into as many equal runs as there are clusters; a run's partial first and last
tile go to scratch as 32-bit partial sums and a second kernel adds up each tile's pieces in run order (a fixed order:
reproducible, int8 exact). Forced here with QGEMM_EVEN_RUNS=1 so that every eligible shape takes it; parity tiers as for
the ordinary path."""
import os

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

SLOT_BYTES = 256 * 256 * 4


def _pair(q):
    return q.Tuning(256, 0, 0, 0, 1, 0)


def _plain(q):
    return q.Tuning(256, 1, 0, 0, 1, 0)  # an explicit split_k = 1 keeps one tile per work item


@pytest.fixture()
def forced(qlib):
    os.environ["QGEMM_EVEN_RUNS"] = "1"
    qlib.lib().qgemm_reload_env()
    yield qlib
    del os.environ["QGEMM_EVEN_RUNS"]
    qlib.lib().qgemm_reload_env()


# 39 tiles (runs shorter than a tile), 32 tiles, 80 ragged tiles (runs longer than a tile: whole tiles inside a run),
# 256 tiles of 8 K blocks (runs of 27 blocks: three whole tiles and two partial ones), 16 tiles
@pytest.mark.parametrize("M,N,K", [(768, 3328, 8192), (1024, 2048, 4096), (2500, 2000, 2064), (4096, 4096, 1024),
                                   (1024, 1024, 6144)])
def test_int8_exact(forced, oracle, dev, M, N, K):
    q = forced
    need = q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _pair(q))
    clusters = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, M, N, K, _pair(q))["ctas"] // 2
    assert need == 2 * 74 * SLOT_BYTES and clusters == 74, (need, clusters)
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, _plain(q)) == 0
    ai = datagen.int8_uniform((M, K), seed=K, stream=0)
    bi = datagen.int8_uniform((N, K), seed=K, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.full((M, N), -1, dtype=torch.int32, device=dev)
    ref = torch.full((M, N), -2, dtype=torch.int32, device=dev)
    q.gemm(a, b, acc, b_kmajor=True, tuning=_pair(q))
    q.gemm(a, b, ref, b_kmajor=True, tuning=_plain(q))
    rc, st = q.device_status()
    assert rc == 0, st
    assert torch.equal(acc, ref), "dealt-out runs and whole tiles must agree exactly"
    got = acc.cpu().numpy()
    for m0, m1 in ((0, 8), (M // 2, M // 2 + 8), (M - 8, M)):
        assert np.array_equal(got[m0:m1], oracle.gemm_i8_rows(ai, bi, m0, m1))
    sa, sb = torch.tensor([0.013], device=dev), torch.tensor([0.009], device=dev)
    c1 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    c2 = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, sa, sb, c1, b_kmajor=True, tuning=_pair(q))
    q.mix_gemm(a, b, sa, sb, c2, b_kmajor=True, tuning=_plain(q))
    assert torch.equal(c1.view(torch.int16), c2.view(torch.int16))
    assert q.device_status()[0] == 0


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
@pytest.mark.parametrize("M,N,K", [(768, 3328, 4096), (1000, 2040, 4096)])
def test_float_kinds(forced, oracle, dev, M, N, K, kind):
    q = forced
    dt = q.BF16 if kind == "bf16" else q.FP8_E4M3
    assert q.workspace_query(dt, q.B_K_MAJOR, M, N, K, _pair(q)) == 2 * 74 * SLOT_BYTES
    a32, b32 = datagen.normal((M, K), 5, 0), datagen.normal((N, K), 5, 1)
    tdt = torch.bfloat16 if kind == "bf16" else torch.float8_e4m3fn
    a, b = torch.from_numpy(a32).to(tdt), torch.from_numpy(b32).to(tdt)
    ref = oracle.gemm_f32(a.float().numpy(), b.float().numpy(), True)
    a, b = a.to(dev), b.to(dev)
    for out in (torch.float32, torch.bfloat16):
        c = torch.full((M, N), float("nan"), dtype=out, device=dev)
        q.gemm(a, b, c, b_kmajor=True, tuning=_pair(q))
        got = c.float().cpu().numpy()
        assert np.isfinite(got).all()
        if kind == "fp8":
            assert oracle.max_rel(got, ref) <= 1e-2  # fp8 tier
        else:
            assert oracle.rel_l2(got, ref) <= (1e-3 if out == torch.float32 else 4e-3)  # 16-bit tier
        again = torch.full((M, N), float("nan"), dtype=out, device=dev)
        q.gemm(a, b, again, b_kmajor=True, tuning=_pair(q))
        view = torch.int32 if out == torch.float32 else torch.int16
        assert torch.equal(c.view(view), again.view(view)), "a fixed order of the sums: bit-identical from run to run"
    assert q.device_status()[0] == 0


def test_too_few_k_blocks_keep_whole_tiles(forced):
    q = forced
    even = 2 * 74 * SLOT_BYTES
    # six tiles of 32 K blocks: a run would have two blocks
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, 300, 520, 4096, _pair(q)) != even
    # a whole number of waves: nothing to even out
    assert q.workspace_query(q.INT8, q.B_K_MAJOR, 256 * 2, 256 * 37, 4096, _pair(q)) != even
