"""GEMM on HOST operands: the call a user of the reference harness effectively makes -- host
buffers in, host result out (tests/includes/test_config.h:239-286 allocates on the host, copies to
the device, runs the kernel and copies C back).

``HostGemm`` owns the device buffers for one problem shape and overlaps the three legs on three
streams: B is uploaded (and relaid out to K-major if it arrives row-major) first, then A is
uploaded in row bands; each band's GEMM starts as soon as its rows have landed and its C rows are
downloaded while later bands are still uploading, so a step costs about max(upload, download)
instead of their sum. All device work goes through the C-ABI kernels; nothing here computes.
"""
from __future__ import annotations

import torch

from . import gemm as _gemm_call
from . import mix_gemm as _mix_call
from . import transpose as _transpose_call


class HostGemm:
    def __init__(self, M: int, N: int, K: int, in_dtype, out_dtype, b_kmajor: bool, device, bands: int = 8):
        self.M, self.N, self.K = M, N, K
        self.b_kmajor = b_kmajor
        self.device = torch.device(device)
        self.bands = max(1, min(bands, (M + 127) // 128))
        rows = (M + self.bands - 1) // self.bands
        rows = (rows + 127) // 128 * 128  # whole output tiles per band
        self.band_rows = rows
        self.bands = (M + rows - 1) // rows
        with torch.cuda.device(self.device):
            self.a = torch.empty((M, K), dtype=in_dtype, device=self.device)
            self.b = torch.empty((N, K) if b_kmajor else (K, N), dtype=in_dtype, device=self.device)
            self.bt = None if b_kmajor else torch.empty((N, K), dtype=in_dtype, device=self.device)
            self.c = torch.empty((M, N), dtype=out_dtype, device=self.device)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_compute = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)
        self.kernel_launches_per_call = self.bands + (0 if b_kmajor else 1)
        self.h2d_bytes = self.a.numel() * self.a.element_size() + self.b.numel() * self.b.element_size()
        self.d2h_bytes = self.c.numel() * self.c.element_size()

    def __call__(self, a_host, b_host, c_host, scale_a=None, scale_b=None) -> None:
        """Enqueue one C = A x B with pinned host tensors; returns once everything is enqueued on the
        current stream's dependency chain (synchronise the current stream to wait for c_host)."""
        cur = torch.cuda.current_stream(self.device)
        start = torch.cuda.Event()
        start.record(cur)
        for s in (self.s_in, self.s_compute, self.s_out):
            s.wait_event(start)

        with torch.cuda.stream(self.s_in):
            self.b.copy_(b_host, non_blocking=True)
            ev_b = torch.cuda.Event()
            ev_b.record(self.s_in)
        with torch.cuda.stream(self.s_compute):
            self.s_compute.wait_event(ev_b)
            if self.b_kmajor:
                b_k = self.b
            else:
                _transpose_call(self.b, self.bt)
                b_k = self.bt

        for i in range(self.bands):
            r0 = i * self.band_rows
            r1 = min(self.M, r0 + self.band_rows)
            with torch.cuda.stream(self.s_in):
                self.a[r0:r1].copy_(a_host[r0:r1], non_blocking=True)
                ev_a = torch.cuda.Event()
                ev_a.record(self.s_in)
            with torch.cuda.stream(self.s_compute):
                self.s_compute.wait_event(ev_a)
                if scale_a is None and scale_b is None:
                    _gemm_call(self.a[r0:r1], b_k, self.c[r0:r1], b_kmajor=True)
                else:
                    _mix_call(self.a[r0:r1], b_k, scale_a, scale_b, self.c[r0:r1], b_kmajor=True)
                ev_c = torch.cuda.Event()
                ev_c.record(self.s_compute)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_c)
                c_host[r0:r1].copy_(self.c[r0:r1], non_blocking=True)

        done_in, done_out = torch.cuda.Event(), torch.cuda.Event()
        done_in.record(self.s_in)
        done_out.record(self.s_out)
        cur.wait_event(done_in)
        cur.wait_event(done_out)
