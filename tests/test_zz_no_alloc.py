"""The allocation-free split-K entry point (qgemm_mix_gemm_splitk_static) against the ordinary one.

Some callers cannot allocate device memory at the point where they need a GEMM -- they run in a loop
that must never risk the device-wide synchronisation an allocation can cause, they are embedded in a
host with a memory budget fixed at start-up, or another allocator already owns all of the GPU's memory. For them the library keeps the
split-K partial sums in a fixed array inside the module instead of its growable scratch. That array is
shared by every call and still holds the previous call's data, so this test makes two calls in a row
(the second on a different, smaller problem, which would expose stale partials) and requires both to
equal the ordinary entry point bit for bit. It is collected last so that a failure here cannot hide
the result of any other test.
"""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu


def _int8_case(dev, M, N, K, seed):
    a = torch.from_numpy(datagen.int8_uniform((M, K), seed=seed, stream=0)).to(dev)
    b = torch.from_numpy(datagen.int8_uniform((N, K), seed=seed, stream=1)).to(dev)
    sa, sb = datagen.scale_pair(seed)
    return a, b, torch.tensor([sa], device=dev), torch.tensor([sb], device=dev)


def test_static_scratch_entry_matches_allocating_entry_twice_in_a_row(qlib, oracle, dev):
    q = qlib
    # call 1: int8 -> bf16 with scales, 4 splits, ragged N
    M, N, K, S = 200, 1030, 2048, 4
    a, b, tsa, tsb = _int8_case(dev, M, N, K, seed=41)
    want = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, tsa, tsb, want, b_kmajor=True, tuning=q.Tuning(128, S, 0, 0))
    got = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=dev)
    q.mix_gemm_splitk_static(a, b, tsa, tsb, got, S)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # and against the oracle: exact accumulator, output within one bf16 ulp
    acc = oracle.gemm_i8(a.cpu().numpy(), b.cpu().numpy(), True)
    ref_bits = oracle.scale_cast(acc, float(tsa.item()), float(tsb.item()), oracle.OUT_BF16)
    got_bits = got.view(torch.int16).cpu().numpy().view(np.uint16)
    assert oracle.bf16_ulp_distance(got_bits, ref_bits) <= 1

    # call 2, straight after: smaller problem, different dtype path (int32 out), 3 splits -- the array
    # still holds call 1's partial sums
    M2, N2, K2, S2 = 70, 264, 1152, 3
    a2, b2, _, _ = _int8_case(dev, M2, N2, K2, seed=42)
    want2 = torch.zeros((M2, N2), dtype=torch.int32, device=dev)
    q.gemm(a2, b2, want2, b_kmajor=True, tuning=q.Tuning(128, S2, 0, 0))
    got2 = torch.full((M2, N2), -1, dtype=torch.int32, device=dev)
    q.mix_gemm_splitk_static(a2, b2, None, None, got2, S2)
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    assert np.array_equal(got2.cpu().numpy(), oracle.gemm_i8(a2.cpu().numpy(), b2.cpu().numpy(), True))


def test_static_scratch_entry_fp8_and_limits(qlib, dev):
    q = qlib
    M, N, K, S = 64, 7168, 2048, 4
    a = torch.randn((M, K), device=dev).to(torch.float8_e4m3fn)
    b = torch.randn((N, K), device=dev).to(torch.float8_e4m3fn)
    sa, sb = torch.tensor([0.02], device=dev), torch.tensor([0.03], device=dev)
    want = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    q.mix_gemm(a, b, sa, sb, want, b_kmajor=True, tuning=q.Tuning(128, S, 0, 0))
    for _ in range(2):
        got = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
        q.mix_gemm_splitk_static(a, b, sa, sb, got, S)
        torch.cuda.synchronize()
        assert torch.equal(got, want)

    L = q.lib()
    big_m = q.STATIC_SCRATCH_BYTES // (S * N * 4) + 1  # one row too many for the fixed array
    rc = L.qgemm_mix_gemm_splitk_static(q.FP8_E4M3, q.BF16, a.data_ptr(), K, b.data_ptr(), K, None, None,
                                        want.data_ptr(), N, big_m, N, K, S, None)
    assert rc == q.ERR_WORKSPACE
    rc = L.qgemm_mix_gemm_splitk_static(q.FP8_E4M3, q.BF16, a.data_ptr(), K, b.data_ptr(), K, None, None,
                                        want.data_ptr(), N, M, N, K, 1, None)
    assert rc == q.ERR_INVALID_ARG  # split_k < 2 uses no scratch: use the ordinary entry point
    rc = L.qgemm_mix_gemm_splitk_static(q.FP8_E4M3, q.BF16, a.data_ptr(), K, b.data_ptr(), K, None, None,
                                        want.data_ptr(), N, M, N, K, 17, None)
    assert rc == q.ERR_INVALID_ARG  # more splits than 128-byte K blocks
    rc, st = q.device_status()
    assert rc == 0, st


def test_static_scratch_entry_reports_a_wait_that_ran_out(qlib, oracle, dev):
    """The entry point keeps its own status words inside the module (it may not allocate any). A bounded wait that
    runs out in its kernel must reach the caller through qgemm_device_status like any other: the failure is made on
    the host (the one-shot hook that has the producer leave out one K block's loads), nothing faults, and the next
    call on the same device is right again."""
    q = qlib
    M, N, K, S = 128, 128, 1024, 2  # two CTAs, K blocks 0..3 and 4..7
    a, b, _, _ = _int8_case(dev, M, N, K, seed=43)
    got = torch.zeros((M, N), dtype=torch.int32, device=dev)
    q.mix_gemm_splitk_static(a, b, None, None, got, S)  # set-up call
    assert q.device_status()[0] == q.OK

    q.lib().qgemm_test_arm_skip_load(2)
    q.mix_gemm_splitk_static(a, b, None, None, got, S)
    rc, st = q.device_status()
    assert rc == q.ERR_DEVICE_TIMEOUT
    assert st[0] == 1 and st[1] == 0 and st[2] == 2 and st[3] == 2  # CTA 0's MMA issuer, waiting for K block 2

    assert q.device_status()[0] == q.OK  # cleared
    q.mix_gemm_splitk_static(a, b, None, None, got, S)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy(), oracle.gemm_i8(a.cpu().numpy(), b.cpu().numpy(), True))
    assert q.device_status()[0] == q.OK
