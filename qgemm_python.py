"""``qgemm_python`` -- the module name the reference's packaging promises (setup.py:56,73 builds an extension of this
name; BUILD_README.md:113-122 and the notebook import it) with the torch-level entry points its sources sketch:
``bf16_mm`` / ``int8_mm`` (src/gemm/sm80_gemm_kernel.cu:4-22) and ``fp8_mm`` (src/mix_gemm/hip_mix_gemm_kernel.cpp:
508-516), all taking ``(a, b, a_scale, b_scale, c)``. Everything is the :mod:`qgemm_b200` binding of ``libqgemm.so``;
``fp8_mm`` here is the reference's block-scaled one (scales per row x 128-K block of a and per 128 x 128 block of b,
operands in the layouts the reference passes), the per-matrix-scale form is ``fp8_mm_per_matrix``."""
from qgemm_b200 import bf16_mm, int8_mm  # noqa: F401
from qgemm_b200 import fp8_block_mm as fp8_mm  # noqa: F401
from qgemm_b200 import fp8_mm as fp8_mm_per_matrix  # noqa: F401
from qgemm_b200 import int4_mm, quantize, transpose  # noqa: F401
