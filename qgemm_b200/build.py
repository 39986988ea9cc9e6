"""In-tree build of libqgemm.so (the CUDA kernels plus the C-ABI) with nvcc for sm_100a.

``python -m qgemm_b200.build`` compiles every translation unit under ``csrc/`` in parallel and
links ``qgemm_b200/libqgemm.so``. nvcc cross-compiles, so this works on a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libqgemm.so")
STAMPS_LIB_PATH = os.path.join(HERE, "libqgemm_stamps.so")  # the diagnostic build, beside the product library

SOURCES = ["gemm_f16.cu", "gemm_i8.cu", "gemm_f8.cu", "gemm_kc_f16.cu", "gemm_kc_i8.cu", "gemm_kc_f8.cu", "transpose.cu", "splitk_reduce.cu", "capi.cu", "cxx_api.cu",
           "no_alloc.cu", "gemm_blockscale.cu", "quantize.cu", "peer.cu", "host_gemm.cu", "int4.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _host_compiler_flags():
    # Prefer the system g++: some images export CC/CXX pointing at a compiler without its runtime specs.
    for cand in ("/usr/bin/g++",):
        if os.path.exists(cand):
            return ["-ccbin", cand]
    return []


def _deps_mtime() -> float:
    newest = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            if name.endswith((".cu", ".cuh", ".h")):
                newest = max(newest, os.path.getmtime(os.path.join(root, name)))
    return newest


def _compile(src: str, verbose: bool, defines=(), obj_dir: str = OBJ_DIR) -> str:
    obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, *_host_compiler_flags(), *[f"-D{d}" for d in defines], "-I",
           os.path.join(HERE, "..", "include"), "-c", os.path.join(CSRC, src), "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, stamps: bool = False) -> str:
    """Build libqgemm.so if it is missing or older than any source. Returns its path. ``stamps`` builds the
    diagnostic variant libqgemm_stamps.so instead (-DQGEMM_STAMPS): the lone-CTA GEMM kernel records SM cycle counts
    along its timeline and the library exports qgemm_debug_stamps to read them; load it with QGEMM_LIBRARY=<path>."""
    out_path = STAMPS_LIB_PATH if stamps else LIB_PATH
    if not force and not stamps and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _deps_mtime():
        return LIB_PATH
    obj_dir = OBJ_DIR + ("_stamps" if stamps else "")
    os.makedirs(obj_dir, exist_ok=True)
    defines = ("QGEMM_STAMPS",) if stamps else ()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, defines, obj_dir), SOURCES))
    cmd = [_nvcc(), *ARCH_FLAGS, *_host_compiler_flags(), "-shared", "-o", out_path, *objs, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return out_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, stamps="--stamps" in sys.argv))
