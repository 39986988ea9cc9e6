"""Failure detection without a GPU fault: a bounded wait that runs out.

Every mbarrier wait in the GEMM kernels gives up after about a second, records where, makes all roles of the
CTA leave their loops, frees its tensor memory and returns; the host reads the status words. The failure is
made on the host: an environment variable tells the dispatcher to have the TMA producer leave out the loads
of one K block, so the MMA issuer waits for a shared-memory slot that nothing fills. Nothing traps, faults or
spins without bound, and the context must stay usable -- the test ends with an ordinary GEMM that is checked
against the oracle. A 1-CTA problem keeps the whole episode to one thread block for one second."""
import os

import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_and_context_survives(qlib, oracle, dev):
    q = qlib
    M, N, K = 128, 128, 512  # one 128x128 tile, 4 K blocks of bf16
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=3, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=3, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    lone_cta = q.Tuning(128, 1, 0, 0, -1, 0)
    assert q.device_status()[0] == q.OK

    os.environ["QGEMM_TEST_SKIP_LOAD"] = "2"  # the producer never fills the slot of K block 2
    try:
        q.gemm(a, b, c, b_kmajor=True, tuning=lone_cta)
        rc, st = q.device_status()  # synchronises: the kernel has returned by itself
    finally:
        del os.environ["QGEMM_TEST_SKIP_LOAD"]
    assert rc == q.ERR_DEVICE_TIMEOUT
    code, cta, role, where = st
    assert code == 1 and cta == 0
    assert role == 2 and where == 2  # the MMA issuer, waiting for K block 2

    # the status words were cleared and the device is fine: the same call now gives the right answer
    assert q.device_status()[0] == q.OK
    q.gemm(a, b, c, b_kmajor=True, tuning=lone_cta)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK
