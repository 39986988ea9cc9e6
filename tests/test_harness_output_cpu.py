"""The C++ harness's output format against the reference's OWN result parser.

tests/golden/gemm_benchmark_mixed_bf16.txt is the stdout of `tests/gemm_benchmark mixed bf16` on a B200 (the
reference's "mixed" shape preset). Where the reference tree is available (QGEMM_REFERENCE_DIR, or its usual mount
point) its scripts/benchmark_to_md.py is loaded from there, unmodified, and must read every problem and every row of
that output; elsewhere the test is skipped -- the parser is the reference's file and is not copied here."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FIXTURE = os.path.join(ROOT, "tests", "golden", "gemm_benchmark_mixed_bf16.txt")
PARSER = os.path.join(os.environ.get("QGEMM_REFERENCE_DIR", "/root/reference"), "scripts", "benchmark_to_md.py")


@pytest.mark.skipif(not os.path.exists(PARSER), reason="reference tree not mounted here")
def test_reference_parser_reads_the_harness_output():
    spec = importlib.util.spec_from_file_location("reference_benchmark_to_md", PARSER)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(FIXTURE) as f:
        data, functions = mod.parse_benchmark_output(f.readlines())
    # the eight problems of the reference's "mixed" preset (tests/includes/example_configs.h:35-53), in order
    assert list(data) == ["M=512, N=512, K=512", "M=1024, N=1024, K=1024", "M=2048, N=512, K=1024",
                          "M=4096, N=1024, K=2048", "M=512, N=2048, K=1024", "M=1024, N=4096, K=2048",
                          "M=1024, N=4096, K=1024", "M=4096, N=1024, K=4096"]
    assert functions == ["GEMM_kernel_v1", "GEMM_kernel_v5", "reference_cublas"]
    for problem, rows in data.items():
        assert set(rows) == set(functions), problem
        for name, r in rows.items():
            assert r["correctness"] == "PASS" and r["tflops"] > 0 and r["time_ms"] > 0 and r["speedup"] > 0
    # and its table generator accepts what it parsed
    table = mod.generate_markdown_table(data, functions, "tflops")
    assert "GEMM_kernel_v1" in table and "M=4096, N=1024, K=4096" in table
