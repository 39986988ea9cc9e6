"""Runs the C++ harness (tests/gemm_benchmark.cpp: the library driven through the reference-style
templates of include/gemm.h, checked against host dot products and timed beside cublasGemmEx) and checks
that the reference's own result parser (the row format of tests/includes/test_config.h:137-159) would read it."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "tests", "gemm_benchmark")


def test_cpp_harness(qlib, dev):
    if not os.path.exists(BINARY):
        import __graft_entry__
        __graft_entry__.build()
    res = subprocess.run([BINARY], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert "Benchmark completed successfully!" in res.stdout
    rows, problem = {}, None
    for line in res.stdout.splitlines():
        m = re.match(r"Problem size: M=(\d+), N=(\d+), K=(\d+)", line.strip())
        if m:
            problem = m.groups()
            continue
        parts = line.split()
        if problem and len(parts) >= 7 and parts[4] in ("PASS", "FAIL"):
            float(parts[1]), float(parts[2]), float(parts[6])  # the columns the reference's parser reads
            rows.setdefault(problem, []).append((parts[0], parts[4]))
    assert len(rows) >= 5  # distinct (M, N, K) keys; several precisions share 4096^3 and 1024^3
    for lst in rows.values():
        assert all(v == "PASS" for _, v in lst), lst
        assert any(n.startswith(("GEMM_kernel", "MIX_GEMM")) for n, _ in lst)
    assert res.stdout.count("matrix_transpose<") == 3 and "FAIL" not in res.stdout


@pytest.mark.parametrize("preset,precision,problems", [("small", "fp16", 3), ("mixed", "bf16", 8)])
def test_cpp_harness_reference_presets(qlib, dev, preset, precision, problems):
    """The shape presets of the reference's tests/includes/example_configs.h:8-53, selected on the command line."""
    if not os.path.exists(BINARY):
        import __graft_entry__
        __graft_entry__.build()
    res = subprocess.run([BINARY, preset, precision], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-2000:]
    assert len(re.findall(r"^Problem size: M=", res.stdout, flags=re.M)) == problems
    assert "FAIL" not in res.stdout and res.stdout.count("PASS") >= 3 * problems
    assert subprocess.run([BINARY, "no-such-preset"], capture_output=True).returncode == 2
