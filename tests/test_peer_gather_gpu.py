"""The gathered column-sharded GEMM across two processes: each rank's epilogue stores its column block into
both ranks' full matrices through a mapping of the other process's allocation (qgemm_peer_export /
qgemm_peer_open + qgemm_gemm_multi_dst). Runs with one GPU (both ranks on it) or more (one rank each)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("shape", [(512, 1024, 512), (300, 656, 208)])
def test_two_ranks_leave_the_whole_matrix_on_both(shape):
    assert torch.cuda.is_available()
    M, n_total, K = shape
    world, port = 2, _free_port()
    env = dict(os.environ)
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "peer_gather_worker.py"), str(r), str(world),
                               str(port), str(M), str(n_total), str(K)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=240)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{out[-3000:]}"
        assert "equals_single_gpu True" in out
