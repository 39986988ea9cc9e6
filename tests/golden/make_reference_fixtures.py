"""Generates tests/golden/reference_bf16_gemm.npz by running the REFERENCE project's own GPU
kernels (oracle/_ref, built by oracle/build_ref.sh from the reference sources) on seeded inputs.

Run on a machine with a GPU from the repository root:

    python tests/golden/make_reference_fixtures.py <output-dir>

The fixture holds the bf16 input bit patterns and the fp32 outputs of the reference's
GEMM_kernel_v1 (WMMA) and GEMM_kernel_v3 (ldmatrix + mma.sync) for one shape every reference kernel
supports, plus whether v2 / v4 / v3_1 agree bit-for-bit with them, and one reference transpose.
The CPU tests check the oracle against these vectors.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_gpu  # noqa: E402


def main(out_dir: str) -> None:
    dev = torch.device("cuda:0")
    M, N, K = 512, 128, 192
    rng = np.random.default_rng(20251125)
    a32 = rng.standard_normal((M, K)).astype(np.float32)
    b32 = rng.standard_normal((K, N)).astype(np.float32)
    a = torch.from_numpy(a32).to(dev).to(torch.bfloat16)
    b = torch.from_numpy(b32).to(dev).to(torch.bfloat16)
    outs = {}
    for v in ("v1", "v2", "v3", "v4"):
        c = torch.zeros((M, N), dtype=torch.float32, device=dev)
        ref_gpu.gemm(v, a, b, c)
        outs[v] = c.cpu().numpy()
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    ref_gpu.gemm("v3_1", a, b.t().contiguous(), c)
    outs["v3_1"] = c.cpu().numpy()

    x = torch.from_numpy(rng.standard_normal((128, 96)).astype(np.float32)).to(dev).to(torch.bfloat16)
    y = torch.zeros((96, 128), dtype=torch.bfloat16, device=dev)
    ref_gpu.transpose(x, y)

    np.savez_compressed(
        os.path.join(out_dir, "reference_bf16_gemm.npz"),
        a_bits=a.view(torch.int16).cpu().numpy().view(np.uint16),
        b_bits=b.view(torch.int16).cpu().numpy().view(np.uint16),
        c_v1=outs["v1"], c_v3=outs["v3"],
        v2_equals_v1=np.array(np.array_equal(outs["v2"], outs["v1"])),
        v4_equals_v3=np.array(np.array_equal(outs["v4"], outs["v3"])),
        v3_1_equals_v3=np.array(np.array_equal(outs["v3_1"], outs["v3"])),
        v4_max_abs_diff_v3=np.array(np.abs(outs["v4"] - outs["v3"]).max()),
        v3_1_max_abs_diff_v3=np.array(np.abs(outs["v3_1"] - outs["v3"]).max()),
        t_in_bits=x.view(torch.int16).cpu().numpy().view(np.uint16),
        t_out_bits=y.view(torch.int16).cpu().numpy().view(np.uint16),
    )
    print("wrote", os.path.join(out_dir, "reference_bf16_gemm.npz"))
    for k, v in outs.items():
        print(k, "max|c|", float(np.abs(v).max()), "diff vs v3", float(np.abs(v - outs["v3"]).max()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else ".")
