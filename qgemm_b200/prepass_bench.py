"""Timing of the HBM-bound passes around the GEMM -- quantise (amax + convert), int4 widening and the B relayout --
on one GPU: ``python -m qgemm_b200.prepass_bench [--rows R --cols C --steps S]``. CUDA events, inputs larger than L2
at the default size; one line per pass with microseconds and GB/s of algorithmic bytes (quantise: 2 reads + 1 write
of the matrix; widening: packed bytes in, int8 bytes out; relayout: 1 read + 1 write)."""
from __future__ import annotations

import argparse
import json


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    import torch

    import qgemm_b200 as q
    dev = torch.device("cuda:0")
    R, Cc = args.rows, args.cols

    def timed(fn):
        for _ in range(max(1, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps * 1e3  # us

    out = []
    for in_dt, es in ((torch.float32, 4), (torch.bfloat16, 2)):
        x = torch.randn((R, Cc), device=dev).to(in_dt)
        for name, fn, out_bytes in (
                ("fp8_e4m3", lambda: q.quantize(x, torch.float8_e4m3fn, out=o8), 1.0),
                ("int8", lambda: q.quantize(x, torch.int8, out=oi), 1.0),
                ("int4", lambda: q.quantize_int4(x, out=o4), 0.5)):
            o8 = torch.empty((R, Cc), dtype=torch.float8_e4m3fn, device=dev)
            oi = torch.empty((R, Cc), dtype=torch.int8, device=dev)
            o4 = torch.empty((R, Cc // 2), dtype=torch.uint8, device=dev)
            us = timed(fn)
            byts = R * Cc * (2 * es + out_bytes)
            out.append({"pass": f"quantize {str(in_dt)[6:]} -> {name}", "us": us, "GB/s": byts / us / 1e3})
        del x
    packed = torch.randint(0, 256, (R, Cc // 2), dtype=torch.uint8, device=dev)
    wide = torch.empty((Cc, R), dtype=torch.int8, device=dev)
    b16 = torch.randn((R, Cc), device=dev).to(torch.bfloat16)
    bt = torch.empty((Cc, R), dtype=torch.bfloat16, device=dev)
    b8 = torch.randint(-127, 128, (R, Cc), dtype=torch.int8, device=dev)
    us = timed(lambda: q.transpose(b16, bt))
    out.append({"pass": "relayout (transpose) 2-byte", "us": us, "GB/s": 2 * R * Cc * 2 / us / 1e3})
    us = timed(lambda: q.transpose(b8, wide))
    out.append({"pass": "relayout (transpose) 1-byte", "us": us, "GB/s": 2 * R * Cc / us / 1e3})
    # int4 widening is internal to the int4 GEMM: time the GEMM against the int8 GEMM on the same shape
    n = min(R, Cc)
    a4 = packed[:n, :n // 2].contiguous()
    a8 = b8[:n, :n].contiguous()
    c = torch.empty((n, n), dtype=torch.bfloat16, device=dev)
    s = torch.tensor([0.01], device=dev)
    t4 = timed(lambda: q.int4_mm(a4, a4, s, s, c))
    t8 = timed(lambda: q.int8_mm(a8, a8, s, s, c))
    out.append({"pass": f"int4 widening of both operands of a {n}^3 product (int4 GEMM - int8 GEMM)", "us": t4 - t8,
                "GB/s": 2 * n * n * 1.5 / max(t4 - t8, 1e-9) / 1e3, "int4_gemm_us": t4, "int8_gemm_us": t8})
    rc, st = q.device_status()
    for row in out:
        print(json.dumps(row))
    assert rc == 0, st


if __name__ == "__main__":
    main()
