#!/usr/bin/env bash
# Compiles the reference project's own GPU kernels for this path, from the sources where they lie,
# into oracle/_ref/libqgemm_ref.so. TEST INFRASTRUCTURE: used only to pin the CPU oracle (and the
# CUDA kernels) against what the reference itself computes. Nothing is copied into this repository.
#
# The reference has no sm_100 code path (every entry point is guarded by `#if CUDA_ARCH == 80/89`),
# so its sm89 kernels (WMMA / ldmatrix / mma.sync / cp.async) are compiled to compute_89 PTX, which
# the driver JIT-compiles for the B200 when the library is first used. `-include cstdint` supplies
# a header the reference's src/include/gemm_utils.cuh uses without including.
set -euo pipefail
REF="${QGEMM_REFERENCE_DIR:-/root/reference}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
mkdir -p "$OUT"
NVCC="${NVCC:-/usr/local/cuda/bin/nvcc}"
SRCS=(
  "$REF/src/gemm/sm89_gemm_kernel_v1.cu"
  "$REF/src/gemm/sm89_gemm_kernel_v2.cu"
  "$REF/src/gemm/sm89_gemm_kernel_v3.cu"
  "$REF/src/gemm/sm89_gemm_kernel_v3.1.cu"
  "$REF/src/gemm/sm89_gemm_kernel_v4.cu"
  "$REF/src/transpose/transpose.cu"
)
"$NVCC" -ccbin /usr/bin/g++ -O3 -std=c++17 -gencode arch=compute_89,code=compute_89 \
  -DCUDA_ARCH=89 -DUSE_CUDA -include cstdint --expt-relaxed-constexpr --expt-extended-lambda \
  -Xcompiler -fPIC -Xcompiler -fpermissive -w \
  -I "$REF/include" -I "$REF/src/include" \
  -shared -o "$OUT/libqgemm_ref.so" "${SRCS[@]}" -lcudart
echo "$OUT/libqgemm_ref.so"

# The reference's own benchmark harness, UNMODIFIED, compiled against this repository's include/
# (gemm.h, blas.h) and linked with libqgemm.so instead of the reference's gemm_lib: the drop-in
# check. Needs qgemm_b200/libqgemm.so (python -m qgemm_b200.build).
REPO="$(cd "$HERE/.." && pwd)"
if [ -f "$REPO/qgemm_b200/libqgemm.so" ]; then
  "$NVCC" -ccbin /usr/bin/g++ -std=c++17 -O2 -DUSE_CUDA -w -Wno-deprecated-gpu-targets \
    -I "$REPO/include" -I "$REF/tests" -I "$REF/tests/includes" \
    "$REF/tests/cuda_benchmark.cpp" \
    -L "$REPO/qgemm_b200" -lqgemm -lcublas \
    -Xlinker -rpath -Xlinker '$ORIGIN/../../qgemm_b200' \
    -o "$OUT/cuda_benchmark"
  echo "$OUT/cuda_benchmark"
fi
