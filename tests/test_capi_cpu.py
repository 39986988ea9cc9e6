"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the public
header declares, and its argument validation / planning logic behaves. No compute is launched."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "qgemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qgemm_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(qlib):
    declared = _declared_symbols()
    assert set(declared) == set(qlib.C_ABI_SYMBOLS)
    L = C.CDLL(qlib.LIB_PATH)
    for sym in declared:
        assert hasattr(L, sym), sym


def test_version_and_status_strings(qlib):
    L = qlib.lib()
    assert L.qgemm_version() >= 100
    seen = set()
    for code in range(7):
        s = qlib.status_string(code)
        assert s and s != "unknown status"
        seen.add(s)
    assert len(seen) == 7
    assert qlib.status_string(12345) == "unknown status"


def test_empty_problem_is_ok_without_touching_the_device(qlib):
    L = qlib.lib()
    assert L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, None, 0, None, 0, None, 0, 0, 128, 64, None) == qlib.OK
    assert L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, None, 0, None, 0, None, 0, 128, 0, 64, None) == qlib.OK
    assert L.qgemm_transpose(None, None, 0, 0, 0, 0, 2, None) == qlib.OK


def test_argument_validation_precedes_any_launch(qlib):
    L = qlib.lib()
    # null output / ld too small
    assert L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, 16, 64, 16, 64, None, 128, 128, 128, 64, None) \
        == qlib.ERR_INVALID_ARG
    assert L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, 16, 64, 16, 64, 16, 64, 128, 128, 64, None) \
        == qlib.ERR_INVALID_ARG
    assert L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, 16, 32, 16, 64, 16, 128, 128, 128, 64, None) \
        == qlib.ERR_INVALID_ARG
    # dtype pairs the plain entry point does not take
    assert L.qgemm_gemm(qlib.FP8_E4M3, qlib.BF16, qlib.B_K_MAJOR, 16, 64, 16, 64, 16, 128, 128, 128, 64, None) \
        == qlib.ERR_UNSUPPORTED
    assert L.qgemm_mix_gemm(qlib.INT8, qlib.INT32, qlib.B_K_MAJOR, 16, 64, 16, 64, None, None, 16, 128, 128, 128, 64,
                            None) == qlib.ERR_UNSUPPORTED
    assert L.qgemm_transpose(16, 32, 8, 8, 8, 8, 4, None) == qlib.ERR_UNSUPPORTED
    assert L.qgemm_transpose(16, 32, 8, 8, 4, 8, 2, None) == qlib.ERR_INVALID_ARG


def test_compute_without_a_gpu_fails_loudly(qlib):
    """There is no CPU fallback: on a machine without CUDA a real call returns an error code."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    L = qlib.lib()
    rc = L.qgemm_gemm(qlib.BF16, qlib.FP32, qlib.B_K_MAJOR, 1024, 64, 2048, 64, 4096, 128, 128, 128, 64, None)
    assert rc in (qlib.ERR_CUDA, qlib.ERR_UNSUPPORTED)
    with pytest.raises(qlib.QgemmError):
        qlib.gemm(torch.zeros(8, 8, dtype=torch.bfloat16), torch.zeros(8, 8, dtype=torch.bfloat16),
                  torch.zeros(8, 8))


def test_workspace_planning(qlib):
    # row-major B needs a relaid-out copy: N * round_up(K, 8) * 2 bytes for bf16
    assert qlib.workspace_query(qlib.BF16, qlib.B_ROW_MAJOR, 8192, 8192, 8192) == 8192 * 8192 * 2
    assert qlib.workspace_query(qlib.BF16, qlib.B_K_MAJOR, 8192, 8192, 8192) == 0
    # an explicit split-K whose slices go through scratch adds splits * M * round_up(N, 4) * 4 bytes of partial sums
    t = qlib.Tuning(128, 3, 0, 0)
    assert qlib.workspace_query(qlib.INT8, qlib.B_K_MAJOR, 100, 518, 2048, t) == 3 * 100 * 520 * 4
    # 2, 4 or 8 slices of few tiles are added up inside the launch (clusters): no partial sums in scratch
    t = qlib.Tuning(128, 4, 0, 0)
    assert qlib.workspace_query(qlib.INT8, qlib.B_K_MAJOR, 100, 518, 2048, t) == 0
    # more splits than 128-byte K blocks cannot be honoured: the plan falls back to what exists
    t = qlib.Tuning(128, 64, 0, 0)
    assert qlib.workspace_query(qlib.INT8, qlib.B_K_MAJOR, 128, 128, 256, t) <= 2 * 128 * 128 * 4
    assert qlib.workspace_query(qlib.BF16, qlib.B_K_MAJOR, 0, 8, 8) == 0


def test_plan_query_ex_and_environment_reload(qlib):
    """Planning is host arithmetic: which kernel configuration a shape gets can be asked without a GPU. The QGEMM_*
    variables are read when the library is loaded; qgemm_reload_env reads them again."""
    import os
    q = qlib
    big = q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192)
    assert (big["tile_m"], big["tile_n"], big["ctas_per_tile"], big["split_k"]) == (512, 256, 2, 1)
    assert big["ctas"] == 148
    skinny = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 7168, 2048)
    assert (skinny["tile_n"], skinny["ctas_per_tile"], skinny["a_rows_per_stage"], skinny["ctas"]) == (64, 1, 16, 112)
    assert skinny["balanced_tiles"] == 0  # opt-in
    deep = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 32, 2048, 8192)
    assert deep["split_k"] > 1  # few tile columns, long K: split-K is the planner's own choice here
    os.environ["QGEMM_BALANCE"] = "1"
    try:
        assert q.lib().qgemm_reload_env() == q.OK
        for M, N in ((16, 7168), (64, 7168), (256, 7168), (100, 7000), (128, 2360)):
            plan = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, M, N, 2048)
            m_tiles = -(-M // 128)
            assert plan["balanced_tiles"] > 0 and plan["balanced_tiles"] * m_tiles <= 148, plan
            units, tiles, narrow = -(-N // 16), plan["balanced_tiles"], plan["min_tile_n"] // 16
            wide_tiles = units - tiles * narrow  # tiles one unit wider than the narrowest
            assert 0 <= wide_tiles < tiles and narrow >= 2
            assert (narrow + (1 if wide_tiles else 0)) * 16 <= plan["tile_n"]  # the kernel's widest tile covers them
    finally:
        del os.environ["QGEMM_BALANCE"]
        q.lib().qgemm_reload_env()
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 7168, 2048)["balanced_tiles"] == 0


def test_plan_in_cluster_split_k(qlib):
    """Few 64- or 128-wide tiles and a long K: the planner cuts K into 2, 4 or 8 slices that the CTAs of one cluster add up
    inside one launch (cluster_slices), as many as still fit the device in one wave. Without a device the number of
    clusters that run at once is taken as seven eighths of SMs / slices."""
    import os
    q = qlib
    for dt in (q.FP8_E4M3, q.BF16, q.INT8):
        deep = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 32, 2048, 8192)  # 32 tiles: four slices = 128 CTAs
        assert (deep["tile_n"], deep["split_k"], deep["cluster_slices"], deep["ctas"]) == (64, 4, 4, 128), deep
        # 64 tiles of 64 columns in two slices, or (taken: fewer bytes per CTA) 32 tiles of 128 columns in four
        four = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 32, 4096, 4096)
        assert (four["tile_n"], four["split_k"], four["cluster_slices"], four["a_rows_per_stage"], four["ctas"]) == (128, 4, 4, 32, 128), four
        eight = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 64, 512, 16384)  # 8 tiles: eight slices
        assert (eight["split_k"], eight["cluster_slices"]) == (8, 8), eight
    # more tiles than half the SMs, or a short K: no slices
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 7168, 2048)["cluster_slices"] == 0
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 128, 1024, 512)["split_k"] == 1
    # a row-major B that is read in place, a CTA cap, or the switch: the slices go through scratch, or there are none
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 32, 2048, 8192, q.Tuning(0, 0, 0, 64, 0, 0))["cluster_slices"] == 0
    os.environ["QGEMM_KCLUSTER"] = "0"
    try:
        q.lib().qgemm_reload_env()
        off = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 32, 2048, 8192)
        assert off["cluster_slices"] == 0 and off["split_k"] > 1, off
    finally:
        del os.environ["QGEMM_KCLUSTER"]
        q.lib().qgemm_reload_env()
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 32, 2048, 8192)["cluster_slices"] == 4


def test_plan_k_grouped_loads_and_narrow_pairs(qlib):
    """Two more planning rules that can be asked without a GPU: K blocks per TMA instruction (two with the 64-wide
    tile when K is a whole number of 128-byte blocks and B is K-major; QGEMM_KGROUP overrides), and 256 x 128 tiles on
    CTA pairs for mid-size problems whose tiles run in one wave."""
    import os
    q = qlib
    skinny = q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 7168, 2048)
    assert (skinny["tile_n"], skinny["k_blocks_per_load"]) == (64, 2), skinny
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 16, 7168, 2040)["k_blocks_per_load"] == 1  # K * 2 % 128 != 0
    assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 256, 7168, 2048)["k_blocks_per_load"] == 1  # 128-wide tile
    assert q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 8192, 8192, 8192)["k_blocks_per_load"] == 1  # CTA pairs
    deep = q.plan_query(q.BF16, q.BF16, q.B_K_MAJOR, 32, 2048, 8192)  # the in-cluster split-K kernel groups too
    assert (deep["cluster_slices"], deep["k_blocks_per_load"]) == (4, 2), deep
    os.environ["QGEMM_KGROUP"] = "1"
    try:
        q.lib().qgemm_reload_env()
        assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 16, 7168, 2048)["k_blocks_per_load"] == 1
        os.environ["QGEMM_KGROUP"] = "8"  # 12 stages with 64 rows of A: 8 does not divide them, 4 does
        q.lib().qgemm_reload_env()
        assert q.plan_query(q.FP8_E4M3, q.BF16, q.B_K_MAJOR, 64, 7168, 2048)["k_blocks_per_load"] == 4
    finally:
        del os.environ["QGEMM_KGROUP"]
        q.lib().qgemm_reload_env()
    for dt in (q.BF16, q.FP8_E4M3):
        mid = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 1024, 2048, 8192)
        assert (mid["tile_m"], mid["tile_n"], mid["ctas_per_tile"], mid["split_k"], mid["ctas"]) == (256, 128, 2, 1, 128), mid
        big = q.plan_query(dt, q.BF16, q.B_K_MAJOR, 4096, 4096, 4096)  # several waves: 256 x 256 pairs
        assert (big["tile_m"], big["tile_n"]) == (256, 256), big
    forced = q.plan_query(q.INT8, q.INT32, q.B_K_MAJOR, 4096, 4096, 4096, q.Tuning(128, 1, 0, 0, 1, 0))
    assert (forced["tile_m"], forced["tile_n"], forced["ctas_per_tile"]) == (256, 128, 2), forced
