"""The relayout kernel against the oracle: bit-exact for every shape, alignment and element size."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (1, 200), (200, 1), (7, 9), (64, 64), (64, 32), (65, 63), (128, 128), (127, 129), (300, 77),
          (1000, 333), (256, 512), (2048, 1024), (4096, 4100)]


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dtype", [torch.int8, torch.bfloat16])
def test_transpose_exact(qlib, oracle, dev, rows, cols, dtype):
    rng = np.random.default_rng(rows * 7 + cols)
    if dtype == torch.int8:
        x = rng.integers(-128, 128, (rows, cols)).astype(np.int8)
        xt = torch.from_numpy(x).to(dev)
        y = qlib.transpose(xt).cpu().numpy()
    else:
        x = rng.integers(0, 65536, (rows, cols)).astype(np.uint16)
        xt = torch.from_numpy(x.view(np.int16)).to(dev).view(torch.bfloat16)
        y = qlib.transpose(xt).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(y, oracle.transpose(x))


def test_transpose_with_leading_dimensions_and_offsets(qlib, oracle, dev):
    """Strided views with odd offsets take the guarded element path; padding stays untouched."""
    rng = np.random.default_rng(1)
    rows, cols = 130, 71
    x = rng.integers(-128, 128, (rows, cols)).astype(np.int8)
    src = torch.zeros((rows, 100), dtype=torch.int8, device=dev)
    src[:, 3:3 + cols] = torch.from_numpy(x).to(dev)
    dst = torch.full((cols, 150), 9, dtype=torch.int8, device=dev)
    qlib.transpose(src[:, 3:3 + cols], dst[:, 5:5 + rows])
    got = dst.cpu().numpy()
    assert np.array_equal(got[:, 5:5 + rows], oracle.transpose(x))
    assert np.all(got[:, :5] == 9) and np.all(got[:, 5 + rows:] == 9)


def test_transpose_involution_at_full_size(qlib, dev):
    """transpose(transpose(x)) == x on the 8192 x 8192 bf16 operand of the BF16 configuration."""
    x = torch.randn((8192, 8192), device=dev).to(torch.bfloat16)
    y = qlib.transpose(x)
    assert torch.equal(y, x.t())
    assert torch.equal(qlib.transpose(y), x)


def test_transpose_rejects_bad_arguments(qlib, dev):
    L = qlib.lib()
    x = torch.zeros((8, 8), dtype=torch.float32, device=dev)
    assert L.qgemm_transpose(x.data_ptr(), x.data_ptr(), 8, 8, 8, 8, 4, None) == qlib.ERR_UNSUPPORTED
    assert L.qgemm_transpose(x.data_ptr(), x.data_ptr(), 8, 8, 4, 8, 2, None) == qlib.ERR_INVALID_ARG
    assert L.qgemm_transpose(None, None, 0, 8, 8, 8, 2, None) == qlib.OK
