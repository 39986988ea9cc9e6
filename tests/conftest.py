import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.build()
    return o


@pytest.fixture(scope="session")
def qlib():
    """The product library; built in-tree if missing. No fallback: a build failure fails the test."""
    from qgemm_b200 import build as qbuild
    qbuild.build()
    import qgemm_b200
    qgemm_b200.lib()
    return qgemm_b200


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test collected on a machine without CUDA; deselect with -m 'not gpu'")
    return torch.device("cuda:0")
