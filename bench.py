#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (`value`): the BF16 configuration -- M = N = K = 8192, A and B both row-major (so B goes
through the relayout kernel), fp32 accumulate, bf16 output, seeded normal(0,1) inputs. One "step" is one pass of
the hot path (relayout + GEMM) over that problem. With N > 1 (launched by torch.distributed.run, one rank per GPU)
every rank runs its own column block of the same width: the global problem is M x (N*8192) x K column-sharded
over the ranks with no data-path collective, i.e. weak scaling; `value` is whole-job TFLOPS =
ranks * 2*M*N*K / max-over-ranks time. The step is timed in several regions of K steps spread through the run
(a power-capped part clocks differently early and late in a run); `value` is their median.

The ONE JSON line printed by rank 0 also carries
  * `e2e`: the same metric through the host-buffer call, both copies inside the timed region;
  * `roofline` of the dominant kernel (per-launch CUDA events), SM clocks sampled during the timed regions;
  * `oracle_check`: sampled rows of the result compared with the CPU oracle, outside every timed region;
  * `c5_int8_sharded` (every N): the int8 32768 x 32768 x 8192 product with B and C column-sharded over the ranks
    (strong scaling): GEMM-only time, and for N > 1 the NCCL all-gather of the C slices and the variant whose
    epilogue stores every tile to all ranks' full matrices over NVLink;
  * `configs` (N = 1): a short measurement of each other configuration -- FP16 1024^3, int8 and FP8 8192^3, the
    FP8 skinny-to-square sweep, two few-tiles-long-K shapes (split-K inside one launch) and two mid-size shapes with the
    library's GEMM timed beside them, the block-scaled FP8 GEMM, the
    1- and 2-byte transpose and the quantise pre-pass -- each with its own roofline fraction and oracle check;
  * `cpu_baseline` (N = 1): the CPU restatement of the reference semantics (the reference ships no CPU GEMM).

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

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu
# captures of these workloads with the kernel and tile shape named in `plan`. Not measured by this program: the
# line reports it as `traffic` with `traffic_source` saying so. None where no capture of that workload exists.
NCU_TRAFFIC_BYTES = {
    "c2_bf16_8192": 883.1e6 + 120.8e6,
    "c3_int8_8192": 237.3e6 + 115.2e6,
    "c4_fp8_16": 14.74e6,
    "d1_fp8_deep": 35.67e6,
    "s1_fp8_skinny_wide": 45.2e6,
    "f1_fp8_blockscale": 131.1e6 + 40.1e6,
}

NOMINAL_PEAK_TFLOPS = {"bf16": 2250.0, "fp16": 2250.0, "int8": 4500.0, "fp8": 4500.0}
ELEM_BYTES = {"bf16": 2, "fp16": 2, "int8": 1, "fp8": 1, "fp32": 4}

WORKLOADS = {
    # name: (in, out, M, N, K, b_kmajor, description)
    "c2_bf16_8192": ("bf16", "bf16", 8192, 8192, 8192, False,
                     "BF16 GEMM M=N=K=8192, A,B row-major (B relaid out to K-major), fp32 acc, bf16 out"),
    "c1_fp16_1024": ("fp16", "fp32", 1024, 1024, 1024, True,
                     "FP16 GEMM M=N=K=1024, B col-major [K,N], uniform[-1,1) seed 0, fp32 out"),
    "c3_int8_8192": ("int8", "bf16", 8192, 8192, 8192, True,
                     "int8 mixed GEMM M=N=K=8192, per-matrix scales, int32 acc, bf16 out"),
    "c3_fp8_8192": ("fp8", "bf16", 8192, 8192, 8192, True,
                    "FP8 e4m3 mixed GEMM M=N=K=8192, per-matrix scales amax/448, fp32 acc, bf16 out"),
    "c4_fp8_16": ("fp8", "bf16", 16, 7168, 2048, True, "FP8 e4m3 M=16 N=7168 K=2048, per-matrix scales, bf16 out"),
    "c4_fp8_64": ("fp8", "bf16", 64, 7168, 2048, True, "FP8 e4m3 M=64 N=7168 K=2048"),
    "c4_fp8_256": ("fp8", "bf16", 256, 7168, 2048, True, "FP8 e4m3 M=256 N=7168 K=2048"),
    "c4_fp8_1024": ("fp8", "bf16", 1024, 7168, 2048, True, "FP8 e4m3 M=1024 N=7168 K=2048"),
    "c4_fp8_6144": ("fp8", "bf16", 6144, 7168, 2048, True, "FP8 e4m3 M=6144 N=7168 K=2048"),
    "f1_fp8_blockscale": ("fp8", "bf16", 4096, 7168, 7168, True,
                          "FP8 e4m3 GEMM with block scales (per row x 128-K block of A, per 128x128 block of B), "
                          "M=4096 N=K=7168, bf16 out: the reference's fp8_mm semantics"),
    "d1_fp8_deep": ("fp8", "bf16", 128, 2048, 16384, True,
                    "FP8 e4m3 M=128 N=2048 K=16384 (few tiles, long K: split-K inside one launch), bf16 out"),
    "d2_bf16_deep": ("bf16", "bf16", 32, 2048, 8192, True, "BF16 M=32 N=2048 K=8192 (few tiles, long K), bf16 out"),
    "s1_fp8_skinny_wide": ("fp8", "bf16", 16, 11008, 4096, True,
                           "FP8 e4m3 M=16 N=11008 K=4096 (too wide for one wave of 64-wide tiles: 128-wide tiles on 16 "
                           "rows of A per stage), bf16 out"),
    "s2_bf16_skinny_wide": ("bf16", "bf16", 8, 28672, 4096, True,
                            "BF16 M=8 N=28672 K=4096 (256-wide tiles on 16 rows of A per stage), bf16 out"),
    "t1_bf16_tail": ("bf16", "bf16", 768, 3328, 8192, True,
                     "BF16 M=768 N=3328 K=8192 (78 tiles of 256 x 128 on 74 CTA pairs: last-wave split), bf16 out"),
    "m1_bf16_mid": ("bf16", "bf16", 1024, 2048, 8192, True,
                    "BF16 M=1024 N=2048 K=8192 (one wave of mid-size tiles: 256 x 128 tiles on CTA pairs), bf16 out"),
    "m2_bf16_mid_deep": ("bf16", "bf16", 1024, 1024, 8192, True,
                         "BF16 M=N=1024 K=8192 (mid-size tiles, long K: K slices of 256 x 128 pair tiles inside one "
                         "launch), bf16 out"),
    "c5_int8_sharded": ("int8", "bf16", 32768, 32768, 8192, True,
                        "int8 mixed GEMM 32768x32768x8192, B/C column-sharded over the ranks (strong scaling)"),
}
CONFIG_BLOCK = ["c1_fp16_1024", "c3_int8_8192", "c3_fp8_8192", "c4_fp8_16", "c4_fp8_64", "c4_fp8_256", "c4_fp8_1024",
                "c4_fp8_6144", "d1_fp8_deep", "d2_bf16_deep", "s1_fp8_skinny_wide", "s2_bf16_skinny_wide", "t1_bf16_tail", "m1_bf16_mid",
                "m2_bf16_mid_deep", "f1_fp8_blockscale"]


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
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps; value = their median")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="never replay the timed loop from a CUDA graph")
    ap.add_argument("--no-like-for-like", action="store_true",
                    help="skip the burst / 3-second sustained timing of the GEMM kernel alone")
    ap.add_argument("--no-c5", action="store_true", help="skip the column-sharded int8 block")
    ap.add_argument("--no-configs", action="store_true", help="skip the short measurements of the other configurations")
    ap.add_argument("--configs", default="", help="comma-separated subset of the other configurations to measure "
                    "(names of WORKLOADS, or hbm_passes); default: all of them")
    ap.add_argument("--no-gather", action="store_true", help="c5, N > 1: skip the all-gather and fused-gather timings")
    ap.add_argument("--stamps", action="store_true",
                    help="diagnostic library only (python -m qgemm_b200.build --stamps, then "
                         "QGEMM_LIBRARY=qgemm_b200/libqgemm_stamps.so): add the lone-CTA kernel's cycle stamps of the "
                         "last launch of the primary workload to the line")
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    return ap.parse_args()


def config_of(workload: str, world: int, seed: int) -> dict:
    """The `config` object, identical for both arms."""
    _, _, M, N, K, _, desc = WORKLOADS[workload]
    if workload == "c5_int8_sharded":
        N = N // world
    return {"workload": workload, "description": desc, "per_rank_shape": [M, N, K], "seed": seed,
            "sharding": f"columns of B/C over {world} rank(s), no data-path collective"}


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while a region is active."""

    def __init__(self, torch_device_index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._active = threading.Event()
        self._thread = None
        self._h = None
        self._mark = 0
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

    def _sample(self):
        nv = self._nv
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

    def _run(self):
        while not self._stop.is_set():
            if self._active.is_set():
                self._sample()
            time.sleep(0.003)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def region(self, on: bool):
        """Switches sampling on / off. Switching off returns the median SM clock seen since it was switched on."""
        if on:
            self._mark = len(self.samples)
            self._active.set()
            return None
        if self._h is not None and self._active.is_set():
            self._sample()  # a region shorter than the sampling period still gets one reading, taken under load
        self._active.clear()
        seen = self.samples[self._mark:]
        return statistics.median(seen) if seen else None

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
    world = int(os.environ.get("WORLD_SIZE", "1"))
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
        "higher_is_better": True, "scaling": "strong" if args.workload == "c5_int8_sharded" else "weak",
        "vs_baseline": None, "dtype": in_name, "data": "synthetic",
        "config": config_of(args.workload, world, args.seed),
        "note": "the reference ships no CPU GEMM; this is the CPU restatement of its semantics, accumulating in "
                + ("int32" if in_name == "int8" else "fp32") + " on the configuration's rounded inputs",
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": arm.threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if ref_gpu_line is not None:
        line["reference_gpu_kernel"] = ref_gpu_line
    emit(line)


# ------------------------------------------------------------------------------------ GPU arm
class Ctx:
    """What every part of the GPU arm needs: the library, the device, the ranks, the clock sampler, the peaks."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import qgemm_b200 as q
        self.torch, self.dist, self.q, self.args = torch, dist, q, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
        self.dev = torch.device("cuda", self.local_rank)
        torch.cuda.set_device(self.dev)
        q.lib()  # fail loudly here if the CUDA library is missing
        self.sampler = ClockSampler(self.local_rank)
        self.sampler.start()
        try:
            self.peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            self.peaks = {}
        self.hbm_peak = float(self.peaks.get("hbm_gbs", 6650.0))
        self.hbm_src = ("measured" if "hbm_gbs" in self.peaks else "fallback") + " copy bandwidth"
        self.dt_code = {"bf16": q.BF16, "fp16": q.FP16, "int8": q.INT8, "fp8": q.FP8_E4M3, "fp32": q.FP32}

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.world > 1:
            t = self.torch.tensor([ms], dtype=self.torch.float64, device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def all_ok(self, ok: bool) -> bool:
        if self.world > 1:
            t = self.torch.tensor([1 if ok else 0], dtype=self.torch.int32, device=self.dev)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
            return bool(t.item())
        return ok

    def event_pair(self):
        return self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)

    def timed(self, step_fn, steps, use_graph=False, sync_ranks=True):
        """Times `steps` calls of step_fn on the current stream with CUDA events, a barrier + synchronize on both
        sides. Returns (milliseconds for all of them on this rank, median SM MHz sampled during the region)."""
        torch = self.torch
        t0, t1 = self.event_pair()
        g = None
        if use_graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(steps):
                    step_fn()
            for _ in range(3):
                g.replay()
        if sync_ranks:
            self.barrier()
        else:
            torch.cuda.synchronize()
        self.sampler.region(True)
        t0.record()
        if g is not None:
            g.replay()
        else:
            for _ in range(steps):
                step_fn()
        t1.record()
        torch.cuda.synchronize()
        mhz = self.sampler.region(False)
        if sync_ranks:
            self.barrier()
        return t0.elapsed_time(t1), mhz


def make_operands(ctx, workload, seed, pin=True):
    """Host and device operands of this rank for one workload. Returns a dict."""
    import numpy as np
    from qgemm_b200 import datagen
    torch, dev, rank, world = ctx.torch, ctx.dev, ctx.rank, ctx.world
    in_name, out_name, M, N, K, b_kmajor, _ = WORKLOADS[workload]
    tdt = {"bf16": torch.bfloat16, "fp16": torch.float16, "int8": torch.int8, "fp8": torch.float8_e4m3fn}[in_name]
    odt = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[out_name]
    if workload == "c5_int8_sharded":
        N = N // world
    sa = sb = sa_h = sb_h = None
    b_stream = 1 + 1000 * rank  # each rank owns different columns of B
    if in_name == "int8":
        a_h = torch.from_numpy(datagen.int8_uniform((M, K), seed, 0))
        b_h = torch.from_numpy(datagen.int8_uniform((N, K) if b_kmajor else (K, N), seed, b_stream))
        s0, s1 = datagen.scale_pair(seed)
        sa_h, sb_h = float(s0), float(s1)
        sa, sb = torch.tensor([s0], device=dev), torch.tensor([s1], device=dev)
    elif in_name == "fp8":
        a32 = torch.from_numpy(datagen.normal((M, K), seed, 0))
        b32 = torch.from_numpy(datagen.normal((N, K) if b_kmajor else (K, N), seed, b_stream))
        s0 = a32.abs().max() / 448.0
        s1 = b32.abs().max() / 448.0
        a_h = (a32 / s0).to(torch.float8_e4m3fn)
        b_h = (b32 / s1).to(torch.float8_e4m3fn)
        sa_h, sb_h = float(s0), float(s1)
        sa, sb = s0.reshape(1).to(dev), s1.reshape(1).to(dev)
        if workload == "f1_fp8_blockscale":  # one scale per (row, 128-K block) of A and per 128x128 block of B
            kbs, nbs = -(-K // 128), -(-N // 128)
            g = torch.Generator().manual_seed(seed)
            sa_h = ((torch.rand((kbs, M), generator=g) * 0.5 + 0.75) * float(s0)).numpy().astype(np.float32)
            sb_h = ((torch.rand((kbs, nbs), generator=g) * 0.5 + 0.75) * float(s1)).numpy().astype(np.float32)
            sa, sb = torch.from_numpy(sa_h).to(dev), torch.from_numpy(sb_h).to(dev)
    else:
        gen = datagen.uniform if workload == "c1_fp16_1024" else datagen.normal
        a_h = torch.from_numpy(gen((M, K), seed, 0)).to(tdt)
        b_h = torch.from_numpy(gen((N, K) if b_kmajor else (K, N), seed, b_stream)).to(tdt)
    c_h = None
    if pin:
        a_h, b_h = a_h.pin_memory(), b_h.pin_memory()
        c_h = torch.empty((M, N), dtype=odt).pin_memory()
    return dict(workload=workload, in_name=in_name, out_name=out_name, M=M, N=N, K=K, a_h=a_h, b_h=b_h, c_h=c_h,
                a=a_h.to(dev), b=b_h.to(dev), c=torch.empty((M, N), dtype=odt, device=dev), sa=sa, sb=sb, sa_h=sa_h,
                sb_h=sb_h, b_kmajor=b_kmajor, in_dtype=tdt, out_dtype=odt,
                blockscale=workload == "f1_fp8_blockscale")


def gemm_call(ctx, ops, a_, b_, c_, b_kmajor, tun):
    q = ctx.q
    if ops["blockscale"]:
        q.fp8_block_mm(a_, b_, ops["sa"], ops["sb"], c_, reference_layout=False)
    else:
        q._gemm(a_, b_, ops["sa"], ops["sb"], c_, b_kmajor, tun, ops["sa"] is not None)


def oracle_check(ctx, ops, c, cols=None, rows=12):
    """Sampled rows of the device result `c` against the CPU oracle (never inside a timed region)."""
    import numpy as np
    torch = ctx.torch
    try:
        from oracle import oracle as o
        from oracle import sampled
        o.set_threads(max(1, (os.cpu_count() or 1) // max(1, ctx.world)))
        a_h, b_h = ops["a_h"], ops["b_h"]
        M = ops["M"]
        in_name = ops["in_name"]
        if in_name == "int8":
            res = sampled.check_int8(a_h.numpy(), b_h.numpy(),
                                     lambda m0, m1: c[m0:m1].contiguous().view(torch.int16).cpu().numpy().view(np.uint16),
                                     "bf16", ops["sa_h"], ops["sb_h"], rows=rows, cols=cols)
        else:
            bt = b_h.float().numpy()
            if not ops["b_kmajor"]:
                bt = np.ascontiguousarray(bt.T)
            a_rows = lambda m0, m1: a_h[m0:m1].float().numpy()
            fetch = lambda m0, m1: c[m0:m1].float().cpu().numpy()
            if ops["blockscale"]:
                res = sampled.check_block_scaled(a_rows, bt, ops["sa_h"], ops["sb_h"], fetch, M, rows=min(rows, 8))
            elif in_name == "fp8":
                res = sampled.check_float(a_rows, bt, fetch, M, "fp8", scale=ops["sa_h"] * ops["sb_h"], rows=rows)
            else:
                res = sampled.check_float(a_rows, bt, fetch, M, "f16", out_16bit=c.element_size() == 2, rows=rows)
        return res
    except Exception as exc:
        return {"ok": False, "error": repr(exc)[:300]}


def roofline_of(ctx, ops, kernel_ms, plan, kernel_name):
    """Roofline object of a GEMM launch: tensor-bound against the measured cuBLAS bf16 burst (16-bit inputs) or the
    nominal dense peak (8-bit inputs: no measured figure exists), HBM-bound below the ridge."""
    in_name = ops["in_name"]
    M, N, K = ops["M"], ops["N"], ops["K"]
    flop = 2.0 * M * N * K
    alg_bytes = (M * K + N * K) * ELEM_BYTES[in_name] + M * N * ELEM_BYTES[ops["out_name"]]
    peaks = ctx.peaks
    if in_name in ("bf16", "fp16"):
        tensor_peak = float(peaks.get("bf16_tflops", 1590.0))
        peak_src = "measured cuBLAS bf16 burst" if "bf16_tflops" in peaks else "fallback 1590"
    else:
        tensor_peak = NOMINAL_PEAK_TFLOPS[in_name]
        peak_src = "nominal dense peak (no measured 8-bit figure exists on this pool)"
    tflops = flop / (kernel_ms * 1e-3) / 1e12
    if flop / alg_bytes < tensor_peak * 1e12 / (ctx.hbm_peak * 1e9):
        gbs = alg_bytes / (kernel_ms * 1e-3) / 1e9
        r = {"bound": "hbm", "achieved": gbs, "peak": ctx.hbm_peak, "unit": "GB/s", "frac": gbs / ctx.hbm_peak,
             "peak_source": ctx.hbm_src, "tflops": tflops}
    else:
        r = {"bound": "tensor", "achieved": tflops, "peak": tensor_peak, "unit": "TFLOP/s",
             "frac": tflops / tensor_peak, "peak_source": peak_src,
             "frac_of_nominal": tflops / NOMINAL_PEAK_TFLOPS[in_name]}
        if in_name in ("bf16", "fp16") and "bf16_tflops_sustained" in peaks:
            r["frac_of_sustained"] = tflops / float(peaks["bf16_tflops_sustained"])
    traffic = NCU_TRAFFIC_BYTES.get(ops["workload"])
    r.update({"kernel": kernel_name, "plan": plan, "kernel_ms": kernel_ms, "algorithmic_flop": flop,
              "algorithmic_bytes": alg_bytes, "traffic": traffic,
              "traffic_source": None if traffic is None else
              "ncu capture of this workload and plan (dram__bytes_read.sum + dram__bytes_write.sum per launch), "
              "not measured in this run"})
    return r


def kernel_name_of(ops, plan):
    if ops["blockscale"]:
        return "fp8_blockscale_kernel"
    if plan.get("cluster_slices", 0) > 1:
        return "gemm_tcgen05_pair_kcluster_kernel" if plan.get("ctas_per_tile") == 2 else "gemm_tcgen05_kcluster_kernel"
    return ("gemm_tcgen05_wide_pair_kernel" if plan["tile_m"] == 512 else
            "gemm_tcgen05_pair_kernel" if plan["ctas_per_tile"] == 2 else "gemm_tcgen05_kernel")


def rotating_sets(ctx, ops):
    """Operands smaller than L2 would be served from L2 on every repeat: enough copies of (A, B, C) that
    consecutive steps never find their inputs cached."""
    torch = ctx.torch
    M, N, K = ops["M"], ops["N"], ops["K"]
    set_bytes = (M * K + N * K) * ELEM_BYTES[ops["in_name"]] + M * N * ops["c"].element_size()
    nsets = 1 if set_bytes > 252e6 else int(min(64, -(-400e6 // set_bytes)))
    sets = [(ops["a"], ops["b"], ops["c"])]
    for _ in range(nsets - 1):
        sets.append((ops["a"].clone(), ops["b"].clone(), torch.empty_like(ops["c"])))
    return sets, set_bytes


def plan_of(ctx, ops, tuning):
    q = ctx.q
    return q.plan_query(ctx.dt_code[ops["in_name"]], ctx.dt_code[ops["out_name"]], q.B_K_MAJOR, ops["M"], ops["N"],
                        ops["K"], tuning)


# ------------------------------------------------------------------------------------ the primary workload
def run_primary(ctx, args):
    torch, q, dev, world = ctx.torch, ctx.q, ctx.dev, ctx.world
    in_name, out_name, M0, N0, K0, _, desc = WORKLOADS[args.workload]
    ops = make_operands(ctx, args.workload, args.seed)
    M, N, K = ops["M"], ops["N"], ops["K"]
    # A row-major B is relaid out to K-major by the transpose kernel, as the BF16 configuration asks; the
    # library's own default for an aligned row-major B (reading it in place) is timed separately below.
    tuning = q.Tuning(args.tile_n, args.split_k, args.group_m, 0, 0, 0 if ops["b_kmajor"] else 1)
    blockscale = ops["blockscale"]
    sets, set_bytes = rotating_sets(ctx, ops)
    nsets = len(sets)
    step_counter = [0]

    def call_device():
        a_, b_, c_ = sets[step_counter[0] % nsets]
        step_counter[0] += 1
        gemm_call(ctx, ops, a_, b_, c_, ops["b_kmajor"], tuning)

    # scratch is reserved before any timed region
    q.workspace_reserve(q.workspace_query(ctx.dt_code[in_name], q.B_K_MAJOR if ops["b_kmajor"] else q.B_ROW_MAJOR,
                                          M, N, K, tuning))
    # Launch-bound workloads (a step of a few microseconds) are replayed from a CUDA graph so that the
    # device, not the Python caller, sets the pace; large steps are launched directly.
    use_graph = (nsets > 1) and not args.no_graph
    flop = 2.0 * M * N * K
    regions = []

    def region(label):
        ms, mhz = ctx.timed(call_device, args.steps, use_graph)
        ms = ctx.max_over_ranks(ms) / args.steps
        regions.append({"after": label, "ms_per_step": ms, "tflops": world * flop / (ms * 1e-3) / 1e12, "sm_mhz": mhz})

    # K-major copies of B: the GEMM kernel on its own (roofline) runs on these
    ksets = sets if ops["b_kmajor"] else [(a_, q.transpose(b_), c_) for a_, b_, c_ in sets]
    kcount = [0]
    relayout_between = not ops["b_kmajor"]

    def call_kernel():
        a_, b_, c_ = ksets[kcount[0] % nsets]
        kcount[0] += 1
        gemm_call(ctx, ops, a_, b_, c_, True, tuning)

    kernel_regions = []

    def kernel_replica():
        """The GEMM kernel's own duration from per-launch events inside a replica of the step loop (for a row-major
        B the relayout launch runs between the timed GEMM launches exactly as it does inside a step, so the kernel
        is timed under the step's own power and clock regime)."""
        for _ in range(3):
            call_kernel()
        torch.cuda.synchronize()
        if use_graph:
            ms, mhz = ctx.timed(call_kernel, args.steps, True, sync_ranks=False)
            kernel_regions.append({"kernel_ms": ms / args.steps, "replica_ms_per_step": None, "sm_mhz": mhz})
            return
        r0, r1 = ctx.event_pair()
        evs = [ctx.event_pair() for _ in range(args.steps)]
        ctx.sampler.region(True)
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
        mhz = ctx.sampler.region(False)
        kernel_regions.append({"kernel_ms": sum(s.elapsed_time(e) for s, e in evs) / len(evs),
                               "replica_ms_per_step": r0.elapsed_time(r1) / len(evs), "sm_mhz": mhz})

    # ---------------- like for like with the measured cuBLAS burst figure: the GEMM kernel alone, best of 10
    # launches timed one by one, taken first, on a GPU that has not been loaded yet (as that figure was), and the
    # library GEMM (torch.matmul, same operands and layout) timed the same way right beside it. Only for the
    # large 16-bit workloads that figure exists for.
    like_for_like = None
    lfl_on = (in_name in ("bf16", "fp16") and nsets == 1 and not args.no_like_for_like and not blockscale
              and ops["c"].dtype == ops["a"].dtype)
    call_library = None
    if lfl_on:
        a0, bk0, c0 = ksets[0]
        lib_out = torch.empty_like(c0)

        def call_library():
            torch.matmul(a0, bk0.t(), out=lib_out)

        def best_of(fn, n):
            best = 1e30
            for _ in range(n):
                b0, b1 = ctx.event_pair()
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
        bu = {"kernel_ms_best_of_10": own_best, "library_ms_best_of_10": lib_best,
              "tflops": flop / (own_best * 1e-3) / 1e12, "library_tflops": flop / (lib_best * 1e-3) / 1e12}
        bu["frac_of_library_same_run"] = bu["tflops"] / bu["library_tflops"]
        if "bf16_tflops" in ctx.peaks:
            bu["peak"] = float(ctx.peaks["bf16_tflops"])
            bu["frac"] = bu["tflops"] / bu["peak"]
        like_for_like = {"burst": bu}

    # ---------------- value: device-resident operands through the public call, in regions spread through the run
    for _ in range(max(args.warmup, 3)):
        call_device()
    n_regions = max(1, args.regions)
    region("warm-up")
    kernel_replica()
    if n_regions >= 2:
        region("kernel replica 1")

    direct_b = None
    if not ops["b_kmajor"]:
        t_direct = q.Tuning(args.tile_n, args.split_k, args.group_m, 0, 0, 0)

        def call_direct():
            a_, b_, c_ = sets[step_counter[0] % nsets]
            step_counter[0] += 1
            q._gemm(a_, b_, ops["sa"], ops["sb"], c_, False, t_direct, ops["sa"] is not None)

        for _ in range(3):
            call_direct()
        # the two paths in alternation, so that both see the same (by now warm, power-capped) GPU
        d_ms, r_ms = 1e30, 1e30
        for _ in range(2):
            d_ms = min(d_ms, ctx.max_over_ranks(ctx.timed(call_direct, args.steps, use_graph)[0]) / args.steps)
            r_ms = min(r_ms, ctx.max_over_ranks(ctx.timed(call_device, args.steps, use_graph)[0]) / args.steps)
        direct_b = {"value": world * flop / (d_ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": d_ms,
                    "relayout_path_same_phase": {"value": world * flop / (r_ms * 1e-3) / 1e12, "ms_per_step": r_ms},
                    "note": "same step with the row-major B read in place as an MN-major tensor-core operand "
                            "(the library default for an aligned B): no relayout pass; timed in alternation with "
                            "the relayout path (best of 2 each)"}
    if n_regions >= 3:
        region("in-place-B comparison" if direct_b else "pause")

    # Like for like with the measured sustained cuBLAS figure (back-to-back launches for seconds, total flops over
    # total time): the GEMM kernel alone and the library GEMM in alternating chunks of 256 launches, about 1.5 s each,
    # so that both run under the same power-capped clock.
    if like_for_like is not None:
        chunk = 256
        tot = {"own": [0.0, 0], "lib": [0.0, 0]}
        while tot["own"][0] + tot["lib"][0] < 3000.0 and tot["own"][1] < 20000:
            for name, fn in (("own", call_kernel), ("lib", call_library)):
                c0e, c1e = ctx.event_pair()
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
        if "bf16_tflops_sustained" in ctx.peaks:
            su["peak"] = float(ctx.peaks["bf16_tflops_sustained"])
            su["frac"] = own_tf / su["peak"]
        like_for_like["sustained"] = su
        like_for_like["library"] = "torch.matmul(A[M,K], B[N,K]^T) -> same dtype as C (cuBLAS), a side figure only"
    kernel_replica()
    if n_regions >= 4:
        region("3 s of back-to-back GEMMs" if like_for_like else "kernel replica 2")

    # the relayout kernel on its own (HBM-bound), when the workload uses it
    relayout = None
    es_in = ELEM_BYTES[in_name]
    if not ops["b_kmajor"]:
        bt = torch.empty((N, K), dtype=ops["in_dtype"], device=dev)
        for _ in range(3):
            q.transpose(ops["b"], bt)
        reps = max(10, args.steps)
        tms = ctx.timed(lambda: q.transpose(ops["b"], bt), reps, False, sync_ranks=False)[0] / reps
        tbytes = 2.0 * N * K * es_in
        relayout = {"kernel": "transpose_kernel", "kernel_ms": tms, "achieved": tbytes / (tms * 1e-3) / 1e9,
                    "peak": ctx.hbm_peak, "unit": "GB/s", "frac": tbytes / (tms * 1e-3) / 1e9 / ctx.hbm_peak,
                    "peak_source": ctx.hbm_src, "algorithmic_bytes": tbytes}

    # ---------------- e2e: host buffers through the host-level call, copies inside the timed region
    e2e = None
    if not args.no_e2e and not blockscale:
        try:
            e2e = run_e2e(ctx, args, ops)
        except Exception as exc:  # the headline must not go down with the host-operand leg
            e2e = {"error": repr(exc)[:300]}
    kernel_replica()
    for i in range(4, n_regions):
        region("host-operand steps" if i == 4 else "pause")

    # ---------------- the result itself against the CPU oracle (sampled rows; outside every timed region)
    gemm_call(ctx, ops, ops["a"], ops["b"], ops["c"], ops["b_kmajor"], tuning)
    torch.cuda.synchronize()
    check = oracle_check(ctx, ops, ops["c"])
    check["ok"] = ctx.all_ok(bool(check.get("ok")))
    check["path"] = "the call timed as `value`, same tuning, every rank's own column block"

    stamps = None
    if args.stamps:
        stamps = read_stamps(ctx)

    ms_list = sorted(r["ms_per_step"] for r in regions)
    ms_per_step = statistics.median(ms_list)
    value = world * flop / (ms_per_step * 1e-3) / 1e12
    kernel_ms = statistics.median(k["kernel_ms"] for k in kernel_regions)
    plan = plan_of(ctx, ops, tuning)
    roofline = roofline_of(ctx, ops, kernel_ms, plan, kernel_name_of(ops, plan))
    roofline["kernel_ms_regions"] = kernel_regions
    if like_for_like is not None and roofline["bound"] == "tensor":
        roofline["like_for_like"] = like_for_like
    launches_per_step = 1 + (0 if ops["b_kmajor"] else 1)
    if q.workspace_query(ctx.dt_code[in_name], q.B_K_MAJOR, M, N, K, tuning) > 0:
        launches_per_step += 1  # split-K / last-wave second pass
    out = {
        "value": value, "ms_per_step": ms_per_step, "dtype": in_name,
        "value_regions": {"n": len(regions), "steps_each": args.steps, "statistic": "median",
                          "min_tflops": min(r["tflops"] for r in regions),
                          "max_tflops": max(r["tflops"] for r in regions), "regions": regions},
        "timing": {"l2": "inputs_larger_than_l2" if nsets == 1 else
                   f"rotating {nsets} operand sets ({nsets * set_bytes / 1e6:.0f} MB) so no step finds its inputs in L2",
                   "timed_loop": "CUDA graph replay" if use_graph else "direct launches"},
        "per_gpu_tflops": value / world, "frac_of_nominal_dense_peak": value / world / NOMINAL_PEAK_TFLOPS[in_name],
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "oracle_check": check,
    }
    if relayout is not None:
        out["relayout_roofline"] = relayout
    if direct_b is not None:
        out["direct_b"] = direct_b
    if stamps is not None:
        out["kernel_timeline_cycles"] = stamps
    return out


def read_stamps(ctx):
    """SM cycle counts along the lone-CTA kernel's timeline (first and last CTA of the last FP8 launch), relative to
    the CTA's entry; only a library built with -DQGEMM_STAMPS exports them."""
    import ctypes as C
    L = ctx.q.lib()
    if not hasattr(L, "qgemm_debug_stamps"):
        return {"unavailable": "the loaded library is not the diagnostic build (QGEMM_LIBRARY)"}
    buf = (C.c_longlong * 32)()
    ctx.torch.cuda.synchronize()
    if L.qgemm_debug_stamps(buf) != 0:
        return {"unavailable": "qgemm_debug_stamps failed"}
    names = ["entry", "set-up done, predecessor complete", "first load issued", "last load issued",
             "first K block landed", "last K block landed", "accumulator committed", "epilogue woke", "epilogue stored"]
    vals = list(buf)
    return {which: {n: vals[base + i] - vals[base] for i, n in enumerate(names)}
            for which, base in (("first_cta", 0), ("last_cta", 16))}


def run_e2e(ctx, args, ops):
    """Host operands in, host result out, through qgemm_gemm_host; both copies inside the timed region. With more
    than one rank the replicated A crosses PCIe once in total: rank r uploads rows [r*M/world, (r+1)*M/world) and
    the ranks all-gather the row blocks over NVLink, then each uploads its own columns of B band by band."""
    torch, world = ctx.torch, ctx.world
    from qgemm_b200.host_api import HostGemm
    M, N, K = ops["M"], ops["N"], ops["K"]
    hg = HostGemm(M, N, K, ops["in_dtype"], ops["out_dtype"], ops["b_kmajor"], ctx.dev,
                  shared_a_group=ctx.dist.group.WORLD if world > 1 else None)
    sa_f, sb_f = (ops["sa_h"], ops["sb_h"]) if ops["sa"] is not None else (None, None)
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        hg(ops["a_h"], ops["b_h"], ops["c_h"], sa_f, sb_f)
    ms, _ = ctx.timed(lambda: hg(ops["a_h"], ops["b_h"], ops["c_h"], sa_f, sb_f), e2e_steps, False)
    e2e_ms = ctx.max_over_ranks(ms) / e2e_steps
    # the host result of the last step against the CPU oracle (sampled rows of the host buffer itself)
    check = oracle_check(ctx, ops, ops["c_h"])
    check["ok"] = ctx.all_ok(bool(check.get("ok")))
    out = {"value": world * 2.0 * M * N * K / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
           "h2d_bytes_per_step": hg.h2d_bytes, "d2h_bytes_per_step": hg.d2h_bytes, "ms_per_step": e2e_ms,
           "steps": e2e_steps, "kernel_launches_per_step": hg.kernel_launches_per_call,
           "nvlink_bytes_received_per_step": hg.nvlink_bytes, "a_upload": hg.a_upload, "oracle_check": check}
    # the ceiling the host side sets: the same bytes copied with no GEMM in between
    out["copy_only"] = hg.copy_only(ops["a_h"], ops["b_h"], ops["c_h"], ctx, steps=max(3, e2e_steps // 2))
    return out


# ------------------------------------------------------------------------------------ c5: column-sharded int8
def run_c5(ctx, args):
    """int8 32768 x 32768 x 8192, B and C column-sharded over the ranks, A replicated: GEMM-only time (max over
    ranks), and for more than one rank the NCCL all-gather of the C slices and the GEMM whose epilogue stores each
    tile to every rank's full matrix. Whole-job throughput = 2*M*N_total*K / time: strong scaling."""
    torch, q, dev, world, rank = ctx.torch, ctx.q, ctx.dev, ctx.world, ctx.rank
    from qgemm_b200 import sharding
    name = "c5_int8_sharded"
    _, _, M, n_total, K, _, desc = WORKLOADS[name]
    steps = max(3, min(args.steps, 10))
    ops = make_operands(ctx, name, args.seed, pin=False)
    N = ops["N"]
    n0, n1 = sharding.partition_columns(n_total, world, rank)
    assert n1 - n0 == N
    call = lambda: sharding.sharded_mix_gemm(ops["a"], ops["b"], ops["sa"], ops["sb"], ops["c"])
    q.workspace_reserve(q.workspace_query(q.INT8, q.B_K_MAJOR, M, N, K, None))
    for _ in range(3):
        call()
    ms, mhz = ctx.timed(call, steps)
    ms = ctx.max_over_ranks(ms) / steps
    total_ops = 2.0 * M * n_total * K
    plan = plan_of(ctx, ops, None)
    # every rank checks sampled rows of its own slice next to both of its edges, i.e. either side of every rank boundary
    cols = [(0, 64), (N - 64, N)]
    check = oracle_check(ctx, ops, ops["c"], cols=cols)
    check["ok"] = ctx.all_ok(bool(check.get("ok")))
    out = {"description": desc, "per_rank_shape": [M, N, K], "ranks": world, "scaling": "strong", "steps": steps,
           "gemm_ms_per_step": ms, "whole_job_tops": total_ops / (ms * 1e-3) / 1e12,
           "tops_per_gpu": total_ops / world / (ms * 1e-3) / 1e12,
           "frac_of_nominal_int8_peak": total_ops / world / (ms * 1e-3) / 1e12 / NOMINAL_PEAK_TFLOPS["int8"],
           "plan": plan, "kernel": kernel_name_of(ops, plan), "sm_mhz": mhz, "oracle_check": check,
           "gpu_launches": steps}
    if world > 1 and not args.no_gather:
        slab_bytes = ops["c"].numel() * ops["c"].element_size()
        for _ in range(2):
            sharding.all_gather_slabs(ops["c"])
        gms = ctx.max_over_ranks(ctx.timed(lambda: sharding.all_gather_slabs(ops["c"]), 5)[0]) / 5
        out["nccl_all_gather"] = {"ms": gms, "bytes_received_per_rank": slab_bytes * (world - 1),
                                  "gemm_plus_all_gather_ms": ms + gms,
                                  "receive_gbs_per_rank": slab_bytes * (world - 1) / (gms * 1e-3) / 1e9}
        # the same gathered result with no separate collective: every rank's GEMM epilogue stores its tiles into
        # all ranks' full matrices over NVLink (one launch per rank per step)
        full = sharding.GatheredOutput(M, n_total, ops["c"].dtype, dev)
        ctx.barrier()
        fcall = lambda: sharding.sharded_mix_gemm_gather(ops["a"], ops["b"], ops["sa"], ops["sb"], full)
        for _ in range(2):
            fcall()
        fms = ctx.max_over_ranks(ctx.timed(fcall, 5)[0]) / 5
        # this rank's copy of the whole C, next to every rank boundary, against the oracle: the boundary rows of
        # every rank's B slice travel over the process group (a few hundred KB)
        edge = torch.cat([ops["b"][:64], ops["b"][-64:]]).contiguous()
        edges = torch.empty((world,) + tuple(edge.shape), dtype=edge.dtype, device=dev)
        ctx.dist.all_gather_into_tensor(edges.view(world * edge.shape[0], K), edge)
        fops = dict(ops)
        fops["b_h"] = edges.view(world * 128, K).cpu()
        picked = torch.cat([full.local[:, r * N + o:r * N + o + 64] for r in range(world) for o in (0, N - 64)], dim=1)
        fcheck = oracle_check(ctx, fops, picked)
        fcheck["ok"] = ctx.all_ok(bool(fcheck.get("ok")))
        fcheck["columns"] = "the 64 columns either side of every rank boundary of this rank's full [M, N] matrix"
        del picked
        full.close()
        out["gemm_with_fused_gather"] = {
            "ms": fms, "launches_per_rank_per_step": 1, "bytes_stored_to_peers_per_rank": slab_bytes * (world - 1),
            "whole_job_tops": total_ops / (fms * 1e-3) / 1e12,
            "frac_of_nvlink_receive_bound": (slab_bytes * (world - 1) / 770e9) / (fms * 1e-3),
            "nvlink_bound": "bytes each GPU must receive / 770 GB/s (measured peer copy, per direction)",
            "oracle_check": fcheck}
        del full
    del ops
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------ the other configurations
def run_config(ctx, args, name):
    """A short measurement of one configuration on one GPU: the step through the public call (graph replay over
    rotating operand sets when the operands fit in L2), its roofline fraction, plan, clocks and oracle check; for
    the FP8 sweep and the two long-K shapes the library's GEMM (torch._scaled_mm / torch.matmul) timed the same way
    beside it."""
    torch, q = ctx.torch, ctx.q
    ops = make_operands(ctx, name, 0 if name == "c1_fp16_1024" else args.seed, pin=False)
    sets, set_bytes = rotating_sets(ctx, ops)
    nsets = len(sets)
    use_graph = nsets > 1 and not args.no_graph
    steps = args.steps if nsets == 1 else max(args.steps, 2 * nsets)
    cnt = [0]

    def call():
        a_, b_, c_ = sets[cnt[0] % nsets]
        cnt[0] += 1
        gemm_call(ctx, ops, a_, b_, c_, True, None)

    q.workspace_reserve(q.workspace_query(ctx.dt_code[ops["in_name"]], q.B_K_MAJOR, ops["M"], ops["N"], ops["K"], None))
    for _ in range(3):
        call()
    best, mhz = 1e30, None
    for _ in range(2):
        ms, m = ctx.timed(call, steps, use_graph, sync_ranks=False)
        if ms / steps < best:
            best, mhz = ms / steps, m
    plan = None if ops["blockscale"] else plan_of(ctx, ops, None)
    roof = roofline_of(ctx, ops, best, plan or {}, kernel_name_of(ops, plan or {"tile_m": 128, "ctas_per_tile": 1}))
    out = {"description": WORKLOADS[name][6], "shape": [ops["M"], ops["N"], ops["K"]], "us": best * 1e3,
           "tflops": roof.get("tflops", roof["achieved"]), "roofline": roof, "sm_mhz": mhz, "steps": steps,
           "timed_loop": ("CUDA graph replay over %d rotating operand sets" % nsets) if use_graph else "direct launches"}
    if name.startswith(("c1_", "c4_", "d1_", "d2_", "m1_", "m2_", "s1_", "s2_", "t1_")) or name == "c3_fp8_8192":
        try:
            lcnt = [0]
            # torch.matmul writes the inputs' type: a 16-bit result buffer of its own where ours is fp32
            lib_out = None
            if ops["in_name"] != "fp8" and ops["c"].dtype != ops["a"].dtype:
                lib_out = torch.empty(ops["c"].shape, dtype=ops["a"].dtype, device=ops["c"].device)

            def lib_call():
                a_, b_, c_ = sets[lcnt[0] % nsets]
                lcnt[0] += 1
                if ops["in_name"] == "fp8":
                    torch._scaled_mm(a_, b_.t(), scale_a=ops["sa"], scale_b=ops["sb"], out_dtype=torch.bfloat16)
                else:
                    torch.matmul(a_, b_.t(), out=c_ if lib_out is None else lib_out)

            for _ in range(3):
                lib_call()
            lbest = min(ctx.timed(lib_call, steps, use_graph, sync_ranks=False)[0] / steps for _ in range(2))
            out["library_scaled_mm_us"] = lbest * 1e3
            out["library"] = ("torch._scaled_mm (cuBLASLt)" if ops["in_name"] == "fp8" else
                              "torch.matmul (cuBLAS)" + ("" if lib_out is None else ", 16-bit out where ours is fp32"))
            out["vs_library"] = lbest / best
        except Exception as exc:
            out["library_scaled_mm_us"] = None
            out["library_error"] = repr(exc)[:160]
    gemm_call(ctx, ops, ops["a"], ops["b"], ops["c"], True, None)
    torch.cuda.synchronize()
    out["oracle_check"] = oracle_check(ctx, ops, ops["c"], rows=8)
    del sets, ops
    torch.cuda.empty_cache()
    return out


def run_hbm_passes(ctx, args):
    """The HBM-bound passes either side of the GEMM: the 2- and 1-byte transpose (relayout) and the quantise pre-pass,
    8192 x 8192 inputs (larger than L2), against the measured copy bandwidth."""
    torch, q, dev = ctx.torch, ctx.q, ctx.dev
    R = Cc = 8192
    out = {}

    def timed(fn, bytes_):
        for _ in range(3):
            fn()
        ms = min(ctx.timed(fn, 20, False, sync_ranks=False)[0] / 20 for _ in range(2))
        gbs = bytes_ / (ms * 1e-3) / 1e9
        return {"us": ms * 1e3, "algorithmic_bytes": bytes_,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": ctx.hbm_peak, "unit": "GB/s",
                             "frac": gbs / ctx.hbm_peak, "peak_source": ctx.hbm_src}}

    b16 = torch.randn((R, Cc), device=dev).to(torch.bfloat16)
    t16 = torch.empty((Cc, R), dtype=torch.bfloat16, device=dev)
    out["transpose_2byte_8192x8192"] = timed(lambda: q.transpose(b16, t16), 2.0 * R * Cc * 2)
    ok16 = bool(torch.equal(t16, b16.t()))
    b8 = torch.randint(-127, 128, (2 * R, Cc), dtype=torch.int8, device=dev)
    t8 = torch.empty((Cc, 2 * R), dtype=torch.int8, device=dev)
    out["transpose_1byte_16384x8192"] = timed(lambda: q.transpose(b8, t8), 2.0 * 2 * R * Cc)
    ok8 = bool(torch.equal(t8, b8.t()))
    out["transpose_exact"] = ok16 and ok8
    del b8, t8, t16
    x32 = torch.randn((R, Cc), device=dev)
    o8 = torch.empty((R, Cc), dtype=torch.float8_e4m3fn, device=dev)
    oi = torch.empty((R, Cc), dtype=torch.int8, device=dev)
    out["quantize_fp32_to_fp8_8192x8192"] = timed(lambda: q.quantize(x32, torch.float8_e4m3fn, out=o8), R * Cc * 9.0)
    out["quantize_bf16_to_int8_8192x8192"] = timed(lambda: q.quantize(b16, torch.int8, out=oi), R * Cc * 5.0)
    out["quantize_bytes"] = "two reads of the input (amax pass, convert pass) + one write of the output"
    del x32, o8, oi, b16
    torch.cuda.empty_cache()
    return out


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

    ctx = Ctx(args)
    torch, q, world, rank = ctx.torch, ctx.q, ctx.world, ctx.rank
    primary = run_primary(ctx, args)

    c5 = None
    if not args.no_c5 and args.workload != "c5_int8_sharded":
        try:
            c5 = run_c5(ctx, args)
        except Exception as exc:  # a side block must not take the headline down with it
            c5 = {"error": repr(exc)[:300]}
    configs = None
    if world == 1 and not args.no_configs:
        configs = {}
        wanted = [n for n in args.configs.split(",") if n] or CONFIG_BLOCK + ["hbm_passes"]
        for name in CONFIG_BLOCK:
            if name == args.workload or name not in wanted:
                continue
            try:
                configs[name] = run_config(ctx, args, name)
            except Exception as exc:
                configs[name] = {"error": repr(exc)[:300]}
        if "hbm_passes" in wanted:
            try:
                configs["hbm_passes"] = run_hbm_passes(ctx, args)
            except Exception as exc:
                configs["hbm_passes"] = {"error": repr(exc)[:300]}

    ctx.sampler.stop()
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
            "metric": "gemm_tflops", "value": primary["value"], "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": primary["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if args.workload == "c5_int8_sharded" else "weak", "vs_baseline": None,
            "dtype": primary["dtype"], "data": "synthetic", "config": config_of(args.workload, world, args.seed),
            "clocks": ctx.sampler.summary(), "cpu_baseline": cpu, "device_status": st if rc else 0,
        }
        for k, v in primary.items():
            if k not in line:
                line[k] = v
        if c5 is not None:
            line["c5_int8_sharded"] = c5
        if configs is not None:
            line["configs"] = configs
        emit(line)
    if world > 1:
        ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
