"""The host-buffer call (qgemm_gemm_host through qgemm_b200.host_api: host operands in, host result out, upload /
compute / download overlapped inside the library) and the library's scratch life cycle."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen
from qgemm_b200.host_api import HostGemm, band_schedule, gemm_host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K,b_kmajor,bands", [(1000, 520, 264, False, 8), (1024, 512, 256, True, 4),
                                                   (130, 256, 128, False, 8), (2048, 1024, 512, True, 3)])
def test_host_gemm_bf16_matches_oracle(qlib, oracle, dev, M, N, K, b_kmajor, bands):
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=M, stream=0))
    b_shape = (N, K) if b_kmajor else (K, N)
    b_bits, b_val = oracle.round_bf16(datagen.normal(b_shape, seed=M, stream=1))
    a_h = torch.from_numpy(a_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
    b_h = torch.from_numpy(b_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
    c_h = torch.zeros((M, N), dtype=torch.float32).pin_memory()
    hg = HostGemm(M, N, K, torch.bfloat16, torch.float32, b_kmajor, dev, bands=bands)
    for _ in range(2):  # the second call reuses every buffer and stream
        c_h.zero_()
        hg(a_h, b_h, c_h)
        torch.cuda.synchronize()
        assert oracle.rel_l2(c_h.numpy(), oracle.gemm_f32(a_val, b_val, b_kmajor)) <= 1e-3
    assert hg.h2d_bytes == (M * K + N * K) * 2 and hg.d2h_bytes == M * N * 4
    assert qlib.device_status()[0] == qlib.OK


def test_host_gemm_int8_scaled(qlib, oracle, dev):
    M, N, K = 700, 384, 512
    ai = datagen.int8_uniform((M, K), seed=1, stream=0)
    bi = datagen.int8_uniform((N, K), seed=1, stream=1)
    sa, sb = datagen.scale_pair(1)
    c_h = torch.zeros((M, N), dtype=torch.bfloat16).pin_memory()
    hg = HostGemm(M, N, K, torch.int8, torch.bfloat16, True, dev)
    hg(torch.from_numpy(ai).pin_memory(), torch.from_numpy(bi).pin_memory(), c_h, torch.tensor([sa], device=dev),
       torch.tensor([sb], device=dev))
    torch.cuda.synchronize()
    ref_bits = oracle.scale_cast(oracle.gemm_i8(ai, bi, True), float(sa), float(sb), oracle.OUT_BF16)
    assert oracle.bf16_ulp_distance(c_h.view(torch.int16).numpy().view(np.uint16), ref_bits) <= 1


def test_host_gemm_pageable_memory_strided_buffers_and_int32(qlib, oracle, dev):
    """Pageable (unpinned) host memory still gives the right answer; host leading dimensions larger than the
    matrix are honoured; INT8 -> INT32 is exact; several column bands and row bands, the last ones ragged."""
    M, N, K = 777, 1300, 400
    ai = datagen.int8_uniform((M, K + 16), seed=4, stream=0)[:, :K]       # lda = K + 16
    bi = datagen.int8_uniform((K, N + 24), seed=4, stream=1)[:, :N]       # row-major B, ldb = N + 24
    a_h, b_h = torch.from_numpy(ai), torch.from_numpy(bi)
    c_full = torch.full((M, N + 8), -7, dtype=torch.int32)
    c_h = c_full[:, :N]                                                    # ldc = N + 8
    assert not a_h.is_contiguous() and not c_h.is_contiguous()
    gemm_host(a_h, b_h, c_h, b_kmajor=False, device=dev)
    torch.cuda.synchronize()
    assert np.array_equal(c_h.numpy(), oracle.gemm_i8(np.ascontiguousarray(ai), np.ascontiguousarray(bi), False))
    assert bool((c_full[:, N:] == -7).all())
    assert qlib.device_status()[0] == qlib.OK


def test_host_gemm_back_to_back_calls_with_different_shapes(qlib, oracle, dev):
    """Calls are enqueued without a host synchronisation in between: the second must not overwrite device
    buffers the first is still using, and a larger problem regrows them."""
    outs = []
    for M, N, K in [(512, 768, 256), (300, 264, 128), (1536, 1024, 512)]:
        a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=K, stream=0))
        b_bits, b_val = oracle.round_bf16(datagen.normal((N, K), seed=K, stream=1))
        a_h = torch.from_numpy(a_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
        b_h = torch.from_numpy(b_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
        c_h = torch.zeros((M, N), dtype=torch.float32).pin_memory()
        gemm_host(a_h, b_h, c_h, b_kmajor=True, device=dev)
        outs.append((c_h, a_val, b_val, a_h, b_h))
    torch.cuda.synchronize()
    for c_h, a_val, b_val, _, _ in outs:
        assert oracle.rel_l2(c_h.numpy(), oracle.gemm_f32(a_val, b_val, True)) <= 1e-3


def test_host_gemm_empty_and_bad_arguments(qlib, dev):
    z = torch.zeros((0, 8), dtype=torch.int8)
    gemm_host(z, torch.zeros((8, 16), dtype=torch.int8), torch.zeros((0, 16), dtype=torch.int32), device=dev)  # M = 0
    c_h = torch.full((4, 16), 5, dtype=torch.int32)
    gemm_host(torch.zeros((4, 0), dtype=torch.int8), torch.zeros((0, 16), dtype=torch.int8), c_h, device=dev)  # K = 0
    torch.cuda.synchronize()
    assert bool((c_h == 0).all())
    with pytest.raises(qlib.QgemmError):
        gemm_host(torch.zeros((4, 8), dtype=torch.int8), torch.zeros((9, 16), dtype=torch.int8), c_h, device=dev)
    with pytest.raises(qlib.QgemmError):
        gemm_host(torch.zeros((4, 8), dtype=torch.float32), torch.zeros((8, 16), dtype=torch.float32),
                  torch.zeros((4, 16), dtype=torch.float32), device=dev)


def test_band_schedule_tiles_the_extent():
    for extent in (1, 200, 256, 257, 1000, 8192, 32768):
        edges = band_schedule(extent, 8)
        assert edges[0][0] == 0 and edges[-1][1] == extent
        assert all(a[1] == b[0] for a, b in zip(edges, edges[1:])) and all(hi > lo for lo, hi in edges)
        assert edges[-1][1] - edges[-1][0] <= 256 or len(edges) == 1


def test_scratch_grows_on_demand_and_survives_shutdown(qlib, oracle, dev):
    """Scratch is grown when a call needs more than is reserved, and qgemm_shutdown() (what
    blas::blas_destroy() calls) frees it; the next call simply sets everything up again."""
    q = qlib
    q.shutdown()
    assert q.lib().qgemm_workspace_bytes() == 0
    M, N, K = 256, 1030, 2048  # N odd: the row-major B cannot be read in place -> relayout scratch; plus split-K
    ai = datagen.int8_uniform((M, K), seed=2, stream=0)
    bi = datagen.int8_uniform((K, N), seed=2, stream=1)
    a, b = torch.from_numpy(ai).to(dev), torch.from_numpy(bi).to(dev)
    acc = torch.zeros((M, N), dtype=torch.int32, device=dev)
    # three slices: not a cluster size, so the partial sums go through scratch
    q.gemm(a, b, acc, b_kmajor=False, tuning=q.Tuning(128, 3, 0, 0, -1, 0))
    need = q.workspace_query(q.INT8, q.B_ROW_MAJOR, M, N, K, q.Tuning(128, 3, 0, 0, -1, 0))
    assert need >= N * K + 3 * M * 1032 * 4
    assert q.lib().qgemm_workspace_bytes() >= need
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, False))
    q.shutdown()
    assert q.lib().qgemm_workspace_bytes() == 0
    acc.zero_()
    q.gemm(a, b, acc, b_kmajor=False)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, False))
    assert q.device_status()[0] == q.OK


@pytest.mark.parametrize("M,N,K,b_kmajor", [(1000, 2100, 264, False), (512, 1536, 512, True), (130, 300, 128, False)])
def test_host_gemm_with_a_resident_on_the_device(qlib, oracle, dev, M, N, K, b_kmajor):
    """qgemm_gemm_host_resident_a: A already on the device (as after the ranks of a column-sharded product have
    exchanged their shares of it), B from the host band by band, C to the host. Same result as the oracle, and the
    same bits as the call that uploads A itself."""
    from qgemm_b200.host_api import gemm_host_resident_a
    a_bits, a_val = oracle.round_bf16(datagen.normal((M, K), seed=N, stream=0))
    b_shape = (N, K) if b_kmajor else (K, N)
    b_bits, b_val = oracle.round_bf16(datagen.normal(b_shape, seed=N, stream=1))
    a_h = torch.from_numpy(a_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
    b_h = torch.from_numpy(b_bits.view(np.int16)).view(torch.bfloat16).pin_memory()
    c_res = torch.zeros((M, N), dtype=torch.bfloat16).pin_memory()
    c_up = torch.zeros((M, N), dtype=torch.bfloat16).pin_memory()
    a_d = a_h.to(dev)
    for _ in range(2):
        c_res.zero_()
        gemm_host_resident_a(a_d, b_h, c_res, None, None, b_kmajor)
        torch.cuda.synchronize()
        assert oracle.rel_l2(c_res.float().numpy(), oracle.gemm_f32(a_val, b_val, b_kmajor)) <= 4e-3  # bf16 output
    gemm_host(a_h, b_h, c_up, b_kmajor=b_kmajor, device=dev)
    torch.cuda.synchronize()
    # both compute each element as one K loop of the same kernel family; tile shapes may differ between the strips
    assert oracle.rel_l2(c_res.float().numpy(), c_up.float().numpy()) <= 1e-6 or \
        oracle.bf16_ulp_distance(c_res.view(torch.int16).numpy().view(np.uint16),
                                 c_up.view(torch.int16).numpy().view(np.uint16)) <= 1
    L = qlib.lib()
    assert L.qgemm_gemm_host_resident_a(qlib.BF16, qlib.BF16, qlib.B_K_MAJOR, None, K, b_h.data_ptr(), K, None, None,
                                        c_res.data_ptr(), N, M, N, K, None) == qlib.ERR_INVALID_ARG
    assert qlib.device_status()[0] == qlib.OK
