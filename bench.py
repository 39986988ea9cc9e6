#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (N = 1): the BF16 configuration -- M = N = K = 8192, A and B both row-major (so B
goes through the relayout kernel), fp32 accumulate, bf16 output, seeded normal(0,1) inputs. One
"step" is one pass of the hot path (relayout + GEMM) over that problem. With N > 1 (launched by
torch.distributed.run, one rank per GPU) every rank runs its own column block of the same width:
the global problem is M x (N*8192) x K column-sharded over the ranks, with no data-path
collective, i.e. weak scaling. `value` is whole-job TFLOPS = ranks * 2*M*N*K / max-over-ranks time.

Prints ONE JSON line on rank 0 with the throughput of device-resident operands (`value`), the same
metric through the host-buffer call with both copies inside the timed region (`e2e`), the live
roofline of the dominant kernel, SM clocks sampled during the timed regions, and -- at N = 1 -- the
CPU baseline (the CPU restatement of the reference semantics; the reference ships no CPU GEMM).

`--impl reference` times that CPU restatement alone (rank 0 only), on a bounded row band per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum), from the
# ncu captures summarised under profiles/. Keyed by workload; None
# where no capture of that workload exists.
NCU_TRAFFIC_BYTES = {
    "c2_bf16_8192": 883.1e6 + 120.8e6,       # profiles/gemm_tcgen05_wide_pair_bf16_8192.md (mean of its two launches)
    "f1_fp8_blockscale": 131.4e6 + 39.6e6,   # profiles/fp8_blockscale_kernel_4096x7168x7168.md
    "c3_int8_8192": 337.7e6 + 114.2e6,       # profiles/gemm_tcgen05_pair_int8_fp8.md
}

NOMINAL_PEAK_TFLOPS = {"bf16": 2250.0, "fp16": 2250.0, "int8": 4500.0, "fp8": 4500.0}

WORKLOADS = {
    # name: (in, out, M, N, K, b_kmajor, description)
    "c2_bf16_8192": ("bf16", "bf16", 8192, 8192, 8192, False,
                     "BF16 GEMM M=N=K=8192, A,B row-major (B relaid out to K-major), fp32 acc, bf16 out"),
    "c1_fp16_1024": ("fp16", "fp32", 1024, 1024, 1024, True,
                     "FP16 GEMM M=N=K=1024, B col-major [K,N], uniform[-1,1) seed 0, fp32 out"),
    "c3_int8_8192": ("int8", "bf16", 8192, 8192, 8192, True,
                     "int8 mixed GEMM M=N=K=8192, per-matrix scales, int32 acc, bf16 out"),
    "c4_fp8_16": ("fp8", "bf16", 16, 7168, 2048, True, "FP8 e4m3 M=16 N=7168 K=2048, per-matrix scales, bf16 out"),
    "c4_fp8_64": ("fp8", "bf16", 64, 7168, 2048, True, "FP8 e4m3 M=64 N=7168 K=2048"),
    "c4_fp8_256": ("fp8", "bf16", 256, 7168, 2048, True, "FP8 e4m3 M=256 N=7168 K=2048"),
    "c4_fp8_1024": ("fp8", "bf16", 1024, 7168, 2048, True, "FP8 e4m3 M=1024 N=7168 K=2048"),
    "c4_fp8_6144": ("fp8", "bf16", 6144, 7168, 2048, True, "FP8 e4m3 M=6144 N=7168 K=2048"),
    "f1_fp8_blockscale": ("fp8", "bf16", 4096, 7168, 7168, True,
                          "FP8 e4m3 GEMM with block scales (per row x 128-K block of A, per 128x128 block of B), "
                          "M=4096 N=K=7168, bf16 out: the reference's fp8_mm semantics"),
    "c5_int8_sharded": ("int8", "bf16", 32768, 32768, 8192, True,
                        "int8 mixed GEMM 32768x32768x8192, B/C column-sharded over the ranks (strong scaling)"),
}


_REAL_STDOUT = None


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is not None:
        os.write(_REAL_STDOUT, data)
    else:
        sys.stdout.write(data.decode())
        sys.stdout.flush()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="never replay the timed loop from a CUDA graph")
    ap.add_argument("--no-like-for-like", action="store_true",
                    help="skip the burst / 3-second sustained timing of the GEMM kernel alone")
    ap.add_argument("--gather", action="store_true", help="c5: also time the all-gather of the C slices")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    return ap.parse_args()


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while active."""

    def __init__(self, torch_device_index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._active = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(torch_device_index)
            self._nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    _REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)) if hasattr(
                        nv, "nvmlDeviceGetCurrentClocksEventReasons") else int(
                        nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                    for bit, name in self._REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(0.004)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def region(self, on: bool):
        (self._active.set if on else self._active.clear)()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------------------------------ CPU arm
class CpuArm:
    """The CPU restatement of the reference semantics (the reference ships no CPU GEMM) on this
    workload's operands: prepared once, then timed on row bands."""

    def __init__(self, workload: str, seed: int):
        from oracle import oracle as o
        from qgemm_b200 import datagen
        in_name, _, M, N, K, _, _ = WORKLOADS[workload]
        self.N = min(N, 8192)  # one rank's column block of the sharded workload, at most this wide
        self.K = K
        rows = min(M, 8192)
        # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
        o.set_threads(os.cpu_count() or 1)
        self.threads = o.num_threads()
        if in_name == "int8":
            self.bt = datagen.int8_uniform((self.N, K), seed, 1)
            self.a = datagen.int8_uniform((rows, K), seed, 0)
            self.fn = o.gemm_i8_blocked
        else:
            bt = datagen.normal((self.N, K), seed, 1)
            a = datagen.normal((rows, K), seed, 0)
            rnd = {"bf16": lambda x: o.round_bf16(x)[1], "fp16": lambda x: o.round_f16(x)[1],
                   "fp8": lambda x: o.quantize_e4m3(x)[1]}[in_name]
            self.bt, self.a = rnd(bt), rnd(a)
            self.fn = o.gemm_f32_blocked

    def run(self, rows: int):
        """Returns (seconds, flop) for rows [0, rows)."""
        rows = min(rows, self.a.shape[0])
        t0 = time.perf_counter()
        self.fn(self.a[:rows], self.bt)
        return time.perf_counter() - t0, 2.0 * rows * self.N * self.K

    def calibrate(self, target_seconds: float) -> int:
        probe = min(96, self.a.shape[0])
        dt, _ = self.run(probe)
        rows = int(probe * target_seconds / max(dt, 1e-6))
        rows = max(48, rows // 48 * 48)
        return min(rows, self.a.shape[0])


def reference_gpu_kernel(M, N, K):
    """Side figure for the reference arm (not the baseline of record, which is the CPU port): the reference's OWN
    GPU kernel, GEMM_kernel_v3<bf16,float> (its fastest published one), compiled unmodified from its sources
    to compute_89 PTX (oracle/build_ref.sh; the reference has no sm_100 code path) and JIT-run on this GPU on the
    same problem, timed the way its harness does (5 warm-ups, 10 back-to-back launches, CUDA events)."""
    try:
        import torch
        from oracle import ref_gpu
        if not (torch.cuda.is_available() and ref_gpu.available()):
            return None
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        a = torch.randn((M, K), device=dev).to(torch.bfloat16)
        b = torch.randn((K, N), device=dev).to(torch.bfloat16)
        c = torch.empty((M, N), dtype=torch.float32, device=dev)
        for _ in range(5):
            ref_gpu.gemm("v3", a, b, c)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn = ref_gpu.launcher("v3")
        torch.cuda.synchronize()
        e0.record(torch.cuda.default_stream())
        for _ in range(10):
            fn(a.data_ptr(), K, b.data_ptr(), N, c.data_ptr(), N, M, N, K)
        e1.record(torch.cuda.default_stream())
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        return {"kernel": "GEMM_kernel_v3<__nv_bfloat16,float> (reference sm89 source, compute_89 PTX JIT)",
                "ms": ms, "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "output": "fp32"}
    except Exception as exc:  # the side figure must never break the arm
        return {"unavailable": repr(exc)[:200]}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    in_name, out_name, M, N, K, b_kmajor, desc = WORKLOADS[args.workload]
    arm = CpuArm(args.workload, args.seed)
    # size the per-step band so that the whole run stays within about a minute of GEMM time
    rows = arm.calibrate(60.0 / max(1, args.steps + args.warmup))
    for _ in range(args.warmup):
        arm.run(rows)
    t_total, flops = 0.0, 0.0
    for _ in range(args.steps):
        dt, fl = arm.run(rows)
        t_total += dt
        flops += fl
    value = flops / t_total / 1e12
    ref_gpu_line = None
    if args.workload == "c2_bf16_8192":
        ref_gpu_line = reference_gpu_kernel(M, N, K)
    sample = (f"rows 0..{rows} x {arm.N} columns x K={K} of the workload per step, blocked OpenMP "
              f"{'int32' if in_name == 'int8' else 'fp32'} GEMM")
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t_total / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if in_name != "int8" else "int32", "data": "synthetic",
        "config": {"workload": args.workload, "description": desc,
                   "note": "the reference ships no CPU GEMM; this is the CPU restatement of its semantics"},
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": arm.threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if ref_gpu_line is not None:
        line["reference_gpu_kernel"] = ref_gpu_line
    emit(line)


# ------------------------------------------------------------------------------------ GPU arm
def make_operands(workload, seed, rank, world, torch, dev):
    """Host (pinned) and device operands of this rank. Returns a dict."""
    import numpy as np
    from qgemm_b200 import datagen
    in_name, out_name, M, N, K, b_kmajor, _ = WORKLOADS[workload]
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8, "fp8": torch.float8_e4m3fn}[in_name]
    odt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[out_name]
    if workload == "c5_int8_sharded":
        n0 = rank * (N // world)
        N = N // world
    sa = sb = None
    b_stream = 1 + 1000 * rank  # each rank owns different columns of B
    if in_name == "int8":
        a_h = torch.from_numpy(datagen.int8_uniform((M, K), seed, 0))
        b_h = torch.from_numpy(datagen.int8_uniform((N, K) if b_kmajor else (K, N), seed, b_stream))
        s0, s1 = datagen.scale_pair(seed)
        sa, sb = torch.tensor([s0], device=dev), torch.tensor([s1], device=dev)
    elif in_name == "fp8":
        a32 = torch.from_numpy(datagen.normal((M, K), seed, 0))
        b32 = torch.from_numpy(datagen.normal((N, K) if b_kmajor else (K, N), seed, b_stream))
        s0 = a32.abs().max() / 448.0
        s1 = b32.abs().max() / 448.0
        a_h = (a32 / s0).to(torch.float8_e4m3fn)
        b_h = (b32 / s1).to(torch.float8_e4m3fn)
        sa, sb = s0.reshape(1).to(dev), s1.reshape(1).to(dev)
        if workload == "f1_fp8_blockscale":  # one scale per (row, 128-K block) of A and per 128x128 block of B
            kbs, nbs = -(-K // 128), -(-N // 128)
            sa = (torch.rand((kbs, M)) * 0.5 + 0.75).mul_(float(s0)).to(dev)
            sb = (torch.rand((kbs, nbs)) * 0.5 + 0.75).mul_(float(s1)).to(dev)
    else:
        gen = datagen.uniform if workload == "c1_fp16_1024" else datagen.normal
        a_h = torch.from_numpy(gen((M, K), seed, 0)).to(tdt)
        b_h = torch.from_numpy(gen((N, K) if b_kmajor else (K, N), seed, b_stream)).to(tdt)
    a_h, b_h = a_h.pin_memory(), b_h.pin_memory()
    c_h = torch.empty((M, N), dtype=odt).pin_memory()
    return dict(M=M, N=N, K=K, a_h=a_h, b_h=b_h, c_h=c_h, a=a_h.to(dev), b=b_h.to(dev),
                c=torch.empty((M, N), dtype=odt, device=dev), sa=sa, sb=sb, b_kmajor=b_kmajor, in_dtype=tdt,
                out_dtype=odt)


def main():
    args = parse_args()
    # The contract is ONE JSON line on stdout: libraries that print there (NCCL's version banner does) are sent
    # to stderr for the duration of the run, and the line is written to the real stdout at the end.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    import qgemm_b200 as q

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    q.lib()  # fail loudly here if the CUDA library is missing

    in_name, out_name, M0, N0, K0, _, desc = WORKLOADS[args.workload]
    ops = make_operands(args.workload, args.seed, rank, world, torch, dev)
    M, N, K = ops["M"], ops["N"], ops["K"]
    # A row-major B is relaid out to K-major by the transpose kernel, as the BF16 configuration asks; the
    # library's own default for an aligned row-major B (reading it in place) is timed separately below.
    tuning = q.Tuning(args.tile_n, args.split_k, args.group_m, 0, 0, 0 if ops["b_kmajor"] else 1)
    mixed = ops["sa"] is not None
    blockscale = args.workload == "f1_fp8_blockscale"

    def gemm_call(a_, b_, c_, b_kmajor, tun):
        if blockscale:
            q.fp8_block_mm(a_, b_, ops["sa"], ops["sb"], c_, reference_layout=False)
        else:
            q._gemm(a_, b_, ops["sa"], ops["sb"], c_, b_kmajor, tun, mixed)

    # Operands smaller than L2 would be served from L2 on every repeat: rotate through enough copies of
    # (A, B, C) that consecutive steps never find their inputs cached.
    es_in0 = 2 if in_name in ("bf16", "fp16") else 1
    set_bytes = (M * K + N * K) * es_in0 + M * N * ops["c"].element_size()
    nsets = 1 if set_bytes > 252e6 else int(min(64, -(-400e6 // set_bytes)))
    sets = [(ops["a"], ops["b"], ops["c"])]
    for _ in range(nsets - 1):
        sets.append((ops["a"].clone(), ops["b"].clone(), torch.empty_like(ops["c"])))
    step_counter = [0]

    def call_device():
        a_, b_, c_ = sets[step_counter[0] % nsets]
        step_counter[0] += 1
        gemm_call(a_, b_, c_, ops["b_kmajor"], tuning)

    # scratch is reserved before any timed region
    q.workspace_reserve(q.workspace_query({"bf16": q.BF16, "fp16": q.FP16, "int8": q.INT8, "fp8": q.FP8_E4M3}[in_name],
                                          q.B_K_MAJOR if ops["b_kmajor"] else q.B_ROW_MAJOR, M, N, K, tuning))
    sampler = ClockSampler(local_rank)
    sampler.start()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # Launch-bound workloads (a step of a few microseconds) are replayed from a CUDA graph so that the
    # device, not the Python caller, sets the pace; large steps are launched directly.
    use_graph = (nsets > 1) and not args.no_graph

    def run_timed(step_fn, steps):
        """Time `steps` calls of step_fn on the current stream. Returns milliseconds for all of them."""
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if use_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(steps):
                    step_fn()
            for _ in range(3):
                g.replay()
            barrier()
            sampler.region(True)
            t0.record()
            g.replay()
            t1.record()
        else:
            barrier()
            sampler.region(True)
            t0.record()
            for _ in range(steps):
                step_fn()
            t1.record()
        torch.cuda.synchronize()
        sampler.region(False)
        return t0.elapsed_time(t1)

    # K-major copies of B: the GEMM kernel on its own (roofline) runs on these
    ksets = sets if ops["b_kmajor"] else [(a_, q.transpose(b_), c_) for a_, b_, c_ in sets]
    kcount = [0]
    relayout_between = not ops["b_kmajor"]

    def call_kernel():
        a_, b_, c_ = ksets[kcount[0] % nsets]
        kcount[0] += 1
        gemm_call(a_, b_, c_, True, tuning)

    # ---------------- like for like with the measured cuBLAS burst figure: the GEMM kernel alone, best of 10
    # launches timed one by one, taken first, on a GPU that has not been loaded yet (as that figure was), and the
    # library GEMM (torch.matmul, same operands and layout) timed the same way right beside it. Only for the
    # large 16-bit workloads that figure exists for.
    like_for_like = None
    lfl_on = (in_name in ("bf16", "fp16") and nsets == 1 and not args.no_like_for_like and not blockscale
              and ops["c"].dtype == ops["a"].dtype)
    if lfl_on:
        a0, bk0, c0 = ksets[0]
        lib_out = torch.empty_like(c0)

        def call_library():
            torch.matmul(a0, bk0.t(), out=lib_out)

        def best_of(fn, n):
            best = 1e30
            for _ in range(n):
                b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                b0.record()
                fn()
                b1.record()
                torch.cuda.synchronize()
                best = min(best, b0.elapsed_time(b1))
            return best

        for _ in range(3):
            call_kernel()
            call_library()
        own_best, lib_best = 1e30, 1e30
        for _ in range(5):  # alternate so that neither sees a systematically warmer GPU
            own_best = min(own_best, best_of(call_kernel, 2))
            lib_best = min(lib_best, best_of(call_library, 2))
        like_for_like = {"burst": {"kernel_ms_best_of_10": own_best, "library_ms_best_of_10": lib_best}}

    # ---------------- value: device-resident operands, the public call
    for _ in range(max(args.warmup, 3)):
        call_device()
    ms_total = max_over_ranks(run_timed(call_device, args.steps))
    barrier()
    ms_per_step = ms_total / args.steps
    flop_per_step_rank = 2.0 * M * N * K
    value = world * flop_per_step_rank / (ms_per_step * 1e-3) / 1e12
    launches_per_step = 1 + (0 if ops["b_kmajor"] else 1)
    ws_partials = q.workspace_query({"bf16": q.BF16, "fp16": q.FP16, "int8": q.INT8, "fp8": q.FP8_E4M3}[in_name],
                                    q.B_K_MAJOR, M, N, K, tuning)
    if ws_partials > 0:
        launches_per_step += 1  # split-K second pass

    # ---------------- roofline of the dominant kernel: the GEMM kernel's own duration, per-launch events, inside a
    # replica of the step loop (for a row-major B the relayout launch runs between the timed GEMM launches exactly
    # as it does inside a step, so the kernel is timed under the step's own power and clock regime). It runs
    # directly after the timed steps above; `replica_ms_per_step` is this loop's own whole-step time, to be read
    # against ms_per_step: on a power-capped part the clock drifts over seconds, and the two loops see it alike
    # only when they are neighbours.
    for _ in range(3):
        call_kernel()
    torch.cuda.synchronize()
    replica_ms = None
    if use_graph:
        gemm_ms = run_timed(call_kernel, args.steps) / args.steps
    else:
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps)]
        sampler.region(True)
        r0.record()
        for i, (s, e) in enumerate(evs):
            if relayout_between:
                _, b_row, _ = sets[i % nsets]
                q.transpose(b_row, ksets[i % nsets][1])
            s.record()
            call_kernel()
            e.record()
        r1.record()
        torch.cuda.synchronize()
        sampler.region(False)
        gemm_ms = sum(s.elapsed_time(e) for s, e in evs) / len(evs)
        replica_ms = r0.elapsed_time(r1) / len(evs)
    achieved_tflops = flop_per_step_rank / (gemm_ms * 1e-3) / 1e12

    direct_b = None
    if not ops["b_kmajor"]:
        t_direct = q.Tuning(args.tile_n, args.split_k, args.group_m, 0, 0, 0)

        def call_direct():
            a_, b_, c_ = sets[step_counter[0] % nsets]
            step_counter[0] += 1
            q._gemm(a_, b_, ops["sa"], ops["sb"], c_, False, t_direct, mixed)

        for _ in range(3):
            call_direct()
        # the two paths in alternation, so that both see the same (by now warm, power-capped) GPU
        d_ms, r_ms = 1e30, 1e30
        for _ in range(2):
            d_ms = min(d_ms, max_over_ranks(run_timed(call_direct, args.steps)) / args.steps)
            r_ms = min(r_ms, max_over_ranks(run_timed(call_device, args.steps)) / args.steps)
        barrier()
        direct_b = {"value": world * flop_per_step_rank / (d_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": d_ms,
                    "relayout_path_same_phase": {"value": world * flop_per_step_rank / (r_ms * 1e-3) / 1e12,
                                                 "ms_per_step": r_ms},
                    "note": "same step with the row-major B read in place as an MN-major tensor-core operand "
                            "(the library default for an aligned B): no relayout pass; timed in alternation with "
                            "the relayout path (best of 2 each)"}

    es_in = 2 if in_name in ("bf16", "fp16") else 1
    es_out = {"bf16": 2, "fp16": 2, "fp32": 4}[out_name]
    alg_bytes = M * K * es_in + N * K * es_in + M * N * es_out
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    ridge_bound = "tensor"
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    hbm_src = "measured" if "hbm_gbs" in peaks else "fallback"
    intensity = flop_per_step_rank / alg_bytes
    if in_name in ("bf16", "fp16"):
        tensor_peak = float(peaks.get("bf16_tflops", 1590.0))
        peak_src = "measured cuBLAS bf16 burst" if "bf16_tflops" in peaks else "fallback 1590"
    else:
        tensor_peak = NOMINAL_PEAK_TFLOPS[in_name]
        peak_src = "nominal dense peak (no measured 8-bit figure exists on this pool)"
    if intensity < tensor_peak * 1e12 / (hbm_peak * 1e9):
        ridge_bound = "hbm"
    if ridge_bound == "tensor":
        roofline = {"bound": "tensor", "achieved": achieved_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": achieved_tflops / tensor_peak, "peak_source": peak_src,
                    "frac_of_sustained": (achieved_tflops / float(peaks["bf16_tflops_sustained"])
                                          if in_name in ("bf16", "fp16") and "bf16_tflops_sustained" in peaks else None),
                    "frac_of_nominal": achieved_tflops / NOMINAL_PEAK_TFLOPS[in_name]}
    else:
        gbs = alg_bytes / (gemm_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                    "peak_source": hbm_src + " copy bandwidth"}
    # Like for like with the measured sustained cuBLAS figure (back-to-back launches for seconds, total flops over
    # total time): the GEMM kernel alone and the library GEMM in alternating chunks of 256 launches, about 1.5 s each,
    # so that both run under the same power-capped clock.
    if like_for_like is not None and ridge_bound == "tensor":
        flop = flop_per_step_rank
        bu = like_for_like["burst"]
        bu.update({"tflops": flop / (bu["kernel_ms_best_of_10"] * 1e-3) / 1e12,
                   "library_tflops": flop / (bu["library_ms_best_of_10"] * 1e-3) / 1e12})
        bu["frac_of_library_same_run"] = bu["tflops"] / bu["library_tflops"]
        if "bf16_tflops" in peaks:
            bu["peak"] = float(peaks["bf16_tflops"])
            bu["frac"] = bu["tflops"] / bu["peak"]
        chunk = 256
        tot = {"own": [0.0, 0], "lib": [0.0, 0]}
        while tot["own"][0] + tot["lib"][0] < 3000.0 and tot["own"][1] < 20000:
            for name, fn in (("own", call_kernel), ("lib", call_library)):
                c0e, c1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0e.record()
                for _ in range(chunk):
                    fn()
                c1e.record()
                torch.cuda.synchronize()
                tot[name][0] += c0e.elapsed_time(c1e)
                tot[name][1] += chunk
        own_tf = flop * tot["own"][1] / (tot["own"][0] * 1e-3) / 1e12
        lib_tf = flop * tot["lib"][1] / (tot["lib"][0] * 1e-3) / 1e12
        su = {"seconds": (tot["own"][0] + tot["lib"][0]) * 1e-3, "launches": tot["own"][1], "tflops": own_tf,
              "library_tflops": lib_tf, "frac_of_library_same_run": own_tf / lib_tf}
        if "bf16_tflops_sustained" in peaks:
            su["peak"] = float(peaks["bf16_tflops_sustained"])
            su["frac"] = own_tf / su["peak"]
        like_for_like["sustained"] = su
        like_for_like["library"] = "torch.matmul(A[M,K], B[N,K]^T) -> same dtype as C (cuBLAS), a side figure only"
        roofline["like_for_like"] = like_for_like
    plan = q.plan_query({"bf16": q.BF16, "fp16": q.FP16, "int8": q.INT8, "fp8": q.FP8_E4M3}[in_name],
                        {"bf16": q.BF16, "fp16": q.FP16, "fp32": q.FP32}[out_name], q.B_K_MAJOR, M, N, K, tuning)
    gemm_kernel_name = ("gemm_tcgen05_wide_pair_kernel" if plan["tile_m"] == 512 else
                        "gemm_tcgen05_pair_kernel" if plan["ctas_per_tile"] == 2 else "gemm_tcgen05_kernel")
    roofline.update({"kernel": "fp8_blockscale_kernel" if blockscale else gemm_kernel_name, "plan": plan,
                     "kernel_ms": gemm_ms, "replica_ms_per_step": replica_ms, "algorithmic_flop": flop_per_step_rank,
                     "algorithmic_bytes": alg_bytes, "traffic": NCU_TRAFFIC_BYTES.get(args.workload)})

    # the relayout kernel on its own (HBM-bound), when the workload uses it
    relayout = None
    if not ops["b_kmajor"]:
        bt = torch.empty((N, K), dtype=ops["in_dtype"], device=dev)
        for _ in range(3):
            q.transpose(ops["b"], bt)
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(10, args.steps)
        t0.record()
        for _ in range(reps):
            q.transpose(ops["b"], bt)
        t1.record()
        torch.cuda.synchronize()
        tms = t0.elapsed_time(t1) / reps
        tbytes = 2.0 * N * K * es_in
        relayout = {"kernel": "transpose_kernel", "kernel_ms": tms, "achieved": tbytes / (tms * 1e-3) / 1e9,
                    "peak": hbm_peak, "unit": "GB/s", "frac": tbytes / (tms * 1e-3) / 1e9 / hbm_peak,
                    "peak_source": hbm_src + " copy bandwidth", "algorithmic_bytes": tbytes}

    # ---------------- e2e: host buffers through the host-level call, copies inside the timed region
    e2e = None
    if not args.no_e2e and not blockscale:
        from qgemm_b200.host_api import HostGemm
        hg = HostGemm(M, N, K, ops["in_dtype"], ops["out_dtype"], ops["b_kmajor"], dev)
        # the host-operand entry takes its two scales as host floats
        sa_f = float(ops["sa"].item()) if ops["sa"] is not None else None
        sb_f = float(ops["sb"].item()) if ops["sb"] is not None else None
        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            hg(ops["a_h"], ops["b_h"], ops["c_h"], sa_f, sb_f)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.region(True)
        s0.record()
        for _ in range(e2e_steps):
            hg(ops["a_h"], ops["b_h"], ops["c_h"], sa_f, sb_f)
        s1.record()
        torch.cuda.synchronize()
        sampler.region(False)
        barrier()
        e2e_ms = max_over_ranks(s0.elapsed_time(s1)) / e2e_steps
        # the host result of the last step against the device-resident call on the same operands (first and last
        # 64 rows; the two may differ in the last bit of a 16-bit output only if their tile shapes differ)
        nr = min(64, M)
        ref_top = torch.empty((nr, N), dtype=ops["out_dtype"], device=dev)
        ref_bot = torch.empty((nr, N), dtype=ops["out_dtype"], device=dev)
        gemm_call(ops["a"][:nr], ops["b"], ref_top, ops["b_kmajor"], None)
        gemm_call(ops["a"][M - nr:], ops["b"], ref_bot, ops["b_kmajor"], None)
        got = torch.cat([ops["c_h"][:nr], ops["c_h"][M - nr:]]).to(dev).float()
        ref = torch.cat([ref_top, ref_bot]).float()
        tol = float(ref.abs().max()) * 2.0 ** -7
        check = bool((got - ref).abs().max() <= tol)
        e2e = {"value": world * flop_per_step_rank / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
               "h2d_bytes_per_step": hg.h2d_bytes, "d2h_bytes_per_step": hg.d2h_bytes, "ms_per_step": e2e_ms,
               "steps": e2e_steps, "kernel_launches_per_step": hg.kernel_launches_per_call,
               "result_roundtrip_ok": check}

    # ---------------- c5: optional all-gather of the C slices (timed separately)
    gather = None
    if args.gather and world > 1:
        from qgemm_b200 import sharding
        for _ in range(2):
            sharding.all_gather_slabs(ops["c"])
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(5):
            sharding.all_gather_slabs(ops["c"])
        g1.record()
        torch.cuda.synchronize()
        gms = max_over_ranks(g0.elapsed_time(g1)) / 5
        gather = {"ms": gms, "bytes_received_per_rank": ops["c"].numel() * ops["c"].element_size() * (world - 1)}

    # ---------------- c5: the same gathered result with no separate collective: every rank's GEMM epilogue
    # stores its tiles into all ranks' full matrices over NVLink (one launch per rank per step)
    fused = None
    if args.gather and world > 1 and args.workload == "c5_int8_sharded":
        from qgemm_b200 import sharding
        out = sharding.GatheredOutput(M, N * world, ops["c"].dtype, dev)
        barrier()
        for _ in range(2):
            sharding.sharded_mix_gemm_gather(ops["a"], ops["b"], ops["sa"], ops["sb"], out)
        torch.cuda.synchronize()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(5):
            sharding.sharded_mix_gemm_gather(ops["a"], ops["b"], ops["sa"], ops["sb"], out)
        f1.record()
        torch.cuda.synchronize()
        barrier()
        fms = max_over_ranks(f0.elapsed_time(f1)) / 5
        # what the separate all-gather assembles must be what the epilogues left behind
        gemm_call(ops["a"], ops["b"], ops["c"], True, None)
        full = sharding.slabs_to_matrix(sharding.all_gather_slabs(ops["c"]))
        same = bool(torch.equal(full.view(torch.int16), out.local.view(torch.int16)))
        del full
        out.close()
        fused = {"ms": fms, "equals_all_gather": same, "launches_per_rank_per_step": 1,
                 "bytes_stored_to_peers_per_rank": ops["c"].numel() * ops["c"].element_size() * (world - 1),
                 "whole_job_tops": 2.0 * M * (N * world) * K / (fms * 1e-3) / 1e12}

    sampler.stop()
    rc, st = q.device_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        arm = CpuArm(args.workload, args.seed)
        rows = arm.calibrate(12.0)
        dt, fl = arm.run(rows)
        cpu = {"value": fl / dt / 1e12, "unit": "TFLOPS", "cores": arm.threads, "kind": "port",
               "sample": f"rows 0..{rows} of the workload ({dt:.1f} s), blocked OpenMP GEMM restating the reference "
                         "semantics (the reference ships no CPU GEMM)"}

    if rank == 0:
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if args.workload == "c5_int8_sharded" else "weak", "vs_baseline": None,
            "dtype": in_name, "data": "synthetic",
            "config": {"workload": args.workload, "description": desc, "per_rank_shape": [M, N, K],
                       "l2": "inputs_larger_than_l2" if nsets == 1 else
                       f"rotating {nsets} operand sets ({nsets * set_bytes / 1e6:.0f} MB) so no step finds its inputs in L2",
                       "timed_loop": "CUDA graph replay" if use_graph else "direct launches",
                       "seed": args.seed, "sharding": f"columns of B/C over {world} rank(s), no data-path collective"},
            "per_gpu_tflops": value / world,
            "frac_of_nominal_dense_peak": value / world / NOMINAL_PEAK_TFLOPS[in_name],
            "roofline": roofline, "clocks": sampler.summary(), "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps, "cpu_baseline": cpu, "device_status": st if rc else 0,
        }
        if relayout is not None:
            line["relayout_roofline"] = relayout
        if direct_b is not None:
            line["direct_b"] = direct_b
        if gather is not None:
            line["all_gather"] = gather
        if fused is not None:
            line["gemm_with_fused_gather"] = fused
        emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
