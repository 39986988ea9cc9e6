"""Failure detection without a GPU fault: a bounded wait that runs out.

Every mbarrier wait in the GEMM kernels gives up after about a second, records where, makes all roles of the
CTA leave their loops, frees its tensor memory and returns; the host reads the status words. The failure is
made on the host: a one-shot test hook of the C-ABI (qgemm_test_arm_skip_load) tells the dispatcher to have the TMA
producers of the next GEMM leave out the loads of one K block, so the MMA issuer waits for a shared-memory slot that nothing fills. Nothing traps, faults or
spins without bound, and the context must stay usable -- the test ends with an ordinary GEMM that is checked
against the oracle. A 1-CTA problem keeps the whole episode to one thread block for one second."""
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

    q.lib().qgemm_test_arm_skip_load(2)  # one-shot: the producer of the next GEMM never fills the slot of K block 2
    q.gemm(a, b, c, b_kmajor=True, tuning=lone_cta)
    rc, st = q.device_status()  # synchronises: the kernel has returned by itself
    assert rc == q.ERR_DEVICE_TIMEOUT
    code, cta, role, where = st
    assert code == 1 and cta == 0
    assert role == 2 and where == 2  # the MMA issuer, waiting for K block 2

    # the status words were cleared and the device is fine: the same call now gives the right answer
    assert q.device_status()[0] == q.OK
    q.gemm(a, b, c, b_kmajor=True, tuning=lone_cta)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK


def test_cta_pair_leaves_together_when_a_wait_runs_out(qlib, oracle, dev):
    """The same host-made failure on the CTA-pair kernel, one cluster of two CTAs on one 256 x 256 tile: the
    leader's MMA issuer gives up, raises the abort flag of BOTH CTAs (a store into the peer's shared memory), and
    the pair meets at its closing cluster barrier well before the peer's own, longer limits would have run out."""
    import time
    q = qlib
    M, N, K = 256, 256, 512  # one pair tile, 8 K blocks of bf16
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=5, stream=0))
    b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=5, stream=1))
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    c = torch.zeros((M, N), dtype=torch.float32, device=dev)
    pair = q.Tuning(256, 1, 0, 0, 1, 0)  # one 256 x 256 tile = one cluster (256 x 128 tiles would make two)
    assert q.plan_query(q.BF16, q.FP32, q.B_K_MAJOR, M, N, K, pair)["ctas_per_tile"] == 2
    q.gemm(a, b, c, b_kmajor=True, tuning=pair)  # warm: module load and attribute set-up are not part of the timing
    assert q.device_status()[0] == q.OK

    def failing_call(tuning):
        q.lib().qgemm_test_arm_skip_load(2)
        t0 = time.perf_counter()
        q.gemm(a, b, c, b_kmajor=True, tuning=tuning)
        rc, st = q.device_status()
        return rc, st, time.perf_counter() - t0

    # yardstick: the lone-CTA kernel leaves after exactly one wait limit (counted in SM cycles, so about a second)
    lone = q.Tuning(128, 1, 0, 0, -1, 0)
    q.gemm(a, b, c, b_kmajor=True, tuning=lone)
    rc, st, t_lone = failing_call(lone)
    assert rc == q.ERR_DEVICE_TIMEOUT and st[2] == 2 and st[3] == 2

    rc, st, t_pair = failing_call(pair)
    assert rc == q.ERR_DEVICE_TIMEOUT
    code, cta, role, where = st
    assert code == 1 and cta == 0 and role == 2 and where == 2  # the leader's MMA issuer, waiting for K block 2
    # the peer CTA did not sit out its epilogue warps' own doubled limit after the leader had given up
    assert t_pair < 1.5 * t_lone, (t_pair, t_lone)

    # the hook was one-shot and the context is intact
    assert q.device_status()[0] == q.OK
    q.gemm(a, b, c, b_kmajor=True, tuning=pair)
    assert oracle.rel_l2(c.cpu().numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3
    assert q.device_status()[0] == q.OK
