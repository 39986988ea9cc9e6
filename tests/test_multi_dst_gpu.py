"""qgemm_gemm_multi_dst: one GEMM, its result stored to several buffers by the same epilogue.

Single process: all destinations live on the same GPU, which exercises the kernel's fan-out exactly as a
multi-GPU run does (the kernel only sees addresses). The result must equal, bit for bit, what the ordinary
entry point writes, in every destination and nowhere else (the buffers are wider than the block written,
as the column block of a gathered matrix is)."""
import ctypes as C

import numpy as np
import pytest
import torch

import qgemm_b200 as q
from oracle import oracle as o
from qgemm_b200 import datagen

pytestmark = pytest.mark.gpu

# the same kernel configuration the multi-destination call uses: CTA pairs, no split-K
PAIR = q.Tuning(0, 1, 0, 0, 1, 0)


def _dev():
    return torch.device("cuda:0")


def _wide_buffers(n, M, n_total, dtype, fill):
    return [torch.full((M, n_total), fill, dtype=dtype, device=_dev()) for _ in range(n)]


@pytest.mark.parametrize("n_dsts", [1, 2, 3, 8])
@pytest.mark.parametrize("shape", [(512, 512, 256), (300, 328, 208), (96, 520, 1024)])
def test_int8_scaled_bf16_every_destination_matches(n_dsts, shape):
    M, N, K = shape
    n_total, n0 = N + 264, 136  # this call's block sits inside a wider matrix, 16-byte aligned start
    a = torch.from_numpy(datagen.int8_uniform((M, K), seed=11, stream=0)).to(_dev())
    b = torch.from_numpy(datagen.int8_uniform((N, K), seed=11, stream=1)).to(_dev())
    sa = torch.tensor([0.0123], device=_dev())
    sb = torch.tensor([0.0071], device=_dev())
    ref = torch.zeros((M, N), dtype=torch.bfloat16, device=_dev())
    q.mix_gemm(a, b, sa, sb, ref, b_kmajor=True, tuning=PAIR)
    bufs = _wide_buffers(n_dsts, M, n_total, torch.bfloat16, 7.0)
    ptrs = [t.data_ptr() + n0 * 2 for t in bufs]
    q.gemm_multi_dst(a, b, sa, sb, ptrs, n_total, torch.bfloat16, N, b_kmajor=True)
    rc, st = q.device_status()
    assert rc == 0, st
    for t in bufs:
        assert torch.equal(t[:, n0:n0 + N].view(torch.int16), ref.view(torch.int16))
        assert bool((t[:, :n0] == 7.0).all()) and bool((t[:, n0 + N:] == 7.0).all())
    # and against the CPU oracle
    acc = o.gemm_i8(a.cpu().numpy(), b.cpu().numpy(), True)
    want = o.scale_cast(acc, float(sa.item()), float(sb.item()), o.OUT_BF16)
    got = bufs[-1][:, n0:n0 + N].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    assert o.bf16_ulp_distance(got, want) <= 1


def test_int8_exact_int32_to_three_destinations():
    M, N, K = 260, 392, 528
    a = torch.from_numpy(datagen.int8_uniform((M, K), seed=5, stream=0)).to(_dev())
    b = torch.from_numpy(datagen.int8_uniform((N, K), seed=5, stream=1)).to(_dev())
    bufs = _wide_buffers(3, M, N + 8, torch.int32, -1)
    q.gemm_multi_dst(a, b, None, None, [t.data_ptr() + 16 for t in bufs], N + 8, torch.int32, N)
    want = o.gemm_i8(a.cpu().numpy(), b.cpu().numpy(), True)
    for t in bufs:
        assert np.array_equal(t[:, 4:4 + N].cpu().numpy(), want)
        assert bool((t[:, :4] == -1).all()) and bool((t[:, 4 + N:] == -1).all())


@pytest.mark.parametrize("b_kmajor", [True, False])
def test_bf16_fp32_out_row_major_b(b_kmajor):
    M, N, K = 384, 640, 328
    rng = np.random.default_rng(2)
    a_bits, a_val = o.round_bf16(rng.standard_normal((M, K)).astype(np.float32))
    b_shape = (N, K) if b_kmajor else (K, N)
    b_bits, b_val = o.round_bf16(rng.standard_normal(b_shape).astype(np.float32))
    a = torch.from_numpy(a_bits.view(np.int16)).to(_dev()).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(_dev()).view(torch.bfloat16)
    ref = torch.zeros((M, N), dtype=torch.float32, device=_dev())
    q.gemm(a, b, ref, b_kmajor=b_kmajor, tuning=PAIR)
    bufs = _wide_buffers(2, M, N, torch.float32, 0.0)
    q.gemm_multi_dst(a, b, None, None, [t.data_ptr() for t in bufs], N, torch.float32, N, b_kmajor=b_kmajor)
    for t in bufs:
        assert torch.equal(t, ref)
    assert o.rel_l2(bufs[0].cpu().numpy(), o.gemm_f32(a_val, b_val, b_kmajor)) <= 1e-3


def test_fp8_two_destinations():
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("no float8 dtype in this torch")
    M, N, K = 256, 512, 384
    rng = np.random.default_rng(9)
    a = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).to(_dev()).to(torch.float8_e4m3fn)
    b = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32)).to(_dev()).to(torch.float8_e4m3fn)
    sa = torch.tensor([0.5], device=_dev())
    sb = torch.tensor([0.25], device=_dev())
    ref = torch.zeros((M, N), dtype=torch.bfloat16, device=_dev())
    q.mix_gemm(a, b, sa, sb, ref, tuning=PAIR)
    bufs = _wide_buffers(2, M, N, torch.bfloat16, 0.0)
    q.gemm_multi_dst(a, b, sa, sb, [t.data_ptr() for t in bufs], N, torch.bfloat16, N)
    for t in bufs:
        assert torch.equal(t.view(torch.int16), ref.view(torch.int16))


def test_argument_errors():
    M, N, K = 128, 128, 128
    a = torch.zeros((M, K), dtype=torch.int8, device=_dev())
    b = torch.zeros((N, K), dtype=torch.int8, device=_dev())
    buf = torch.zeros((M, N + 8), dtype=torch.bfloat16, device=_dev())
    with pytest.raises(q.QgemmError) as e:  # too many destinations
        q.gemm_multi_dst(a, b, None, None, [buf.data_ptr()] * 9, N + 8, torch.bfloat16, N)
    assert e.value.status == q.ERR_INVALID_ARG
    with pytest.raises(q.QgemmError) as e:  # none
        q.gemm_multi_dst(a, b, None, None, [], N + 8, torch.bfloat16, N)
    assert e.value.status == q.ERR_INVALID_ARG
    with pytest.raises(q.QgemmError) as e:  # a second destination that is not 16-byte aligned
        q.gemm_multi_dst(a, b, None, None, [buf.data_ptr(), buf.data_ptr() + 2], N + 8, torch.bfloat16, N)
    assert e.value.status == q.ERR_ALIGNMENT
    with pytest.raises(q.QgemmError) as e:  # a leading dimension that is not a multiple of 16 bytes
        q.gemm_multi_dst(a, b, None, None, [buf.data_ptr(), buf.data_ptr()], N + 3, torch.bfloat16, N)
    assert e.value.status == q.ERR_ALIGNMENT
    # a null destination, straight through the C-ABI
    arr = (C.c_void_p * 2)(buf.data_ptr(), None)
    rc = q.lib().qgemm_gemm_multi_dst(q.INT8, q.BF16, q.B_K_MAJOR, a.data_ptr(), K, b.data_ptr(), K, None, None, arr,
                                      2, N + 8, M, N, K, None)
    assert rc == q.ERR_INVALID_ARG
    rc, st = q.device_status()
    assert rc == 0, st


def test_empty_k_zeroes_every_destination():
    M, N = 64, 72
    a = torch.zeros((M, 0), dtype=torch.int8, device=_dev())
    b = torch.zeros((N, 0), dtype=torch.int8, device=_dev())
    bufs = _wide_buffers(3, M, N, torch.bfloat16, 3.0)
    arr = (C.c_void_p * 3)(*[t.data_ptr() for t in bufs])
    rc = q.lib().qgemm_gemm_multi_dst(q.INT8, q.BF16, q.B_K_MAJOR, a.data_ptr(), 0, b.data_ptr(), 0, None, None, arr,
                                      3, N, M, N, 0, None)
    assert rc == q.OK
    torch.cuda.synchronize()
    for t in bufs:
        assert bool((t == 0).all())
