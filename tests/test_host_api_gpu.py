"""The host-buffer call (qgemm_b200.host_api.HostGemm: pinned host operands in, host result out, upload /
compute / download overlapped on three streams) and the library's scratch life cycle."""
import numpy as np
import pytest
import torch

from qgemm_b200 import datagen
from qgemm_b200.host_api import HostGemm

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
    q.gemm(a, b, acc, b_kmajor=False, tuning=q.Tuning(128, 4, 0, 0, -1, 0))
    need = q.workspace_query(q.INT8, q.B_ROW_MAJOR, M, N, K, q.Tuning(128, 4, 0, 0, -1, 0))
    assert need >= N * K + 4 * M * 1032 * 4
    assert q.lib().qgemm_workspace_bytes() >= need
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, False))
    q.shutdown()
    assert q.lib().qgemm_workspace_bytes() == 0
    acc.zero_()
    q.gemm(a, b, acc, b_kmajor=False)
    assert np.array_equal(acc.cpu().numpy(), oracle.gemm_i8(ai, bi, False))
    assert q.device_status()[0] == q.OK
