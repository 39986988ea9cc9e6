"""Column sharding across ranks: partition arithmetic, and the gathered slab layout exercised with
real torch.distributed ranks (gloo, world size 2) on CPU. The rank-local GEMM is the ordinary
single-GPU kernel, so on CPU its place is taken by the oracle -- what is under test here is the
sharding and gather logic."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qgemm_b200 import sharding


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partitions_tile_the_columns(world):
    N = 32768
    parts = sharding.all_partitions(N, world)
    assert parts[0][0] == 0 and parts[-1][1] == N
    for (a0, a1), (b0, b1) in zip(parts, parts[1:]):
        assert a1 == b0
    assert len({b - a for a, b in parts}) == 1
    assert parts[0][1] - parts[0][0] == N // world


def test_partition_rejects_ragged_and_bad_ranks():
    with pytest.raises(ValueError):
        sharding.partition_columns(100, 8, 0)
    with pytest.raises(ValueError):
        sharding.partition_columns(128, 4, 4)
    with pytest.raises(ValueError):
        sharding.partition_columns(128, 0, 0)


def test_slabs_to_matrix():
    world, M, n_per = 4, 3, 5
    full = torch.arange(M * world * n_per).reshape(M, world * n_per)
    slabs = torch.stack([full[:, r * n_per:(r + 1) * n_per] for r in range(world)])
    assert torch.equal(sharding.slabs_to_matrix(slabs), full)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, M, N, K, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as o
        from qgemm_b200 import datagen
        a = datagen.int8_uniform((M, K), seed=3, stream=0)       # replicated
        b_full = datagen.int8_uniform((N, K), seed=3, stream=1)  # every rank can regenerate it
        n0, n1 = sharding.partition_columns(N, world, rank)
        acc = o.gemm_i8(a, b_full[n0:n1], True)                  # stand-in for the rank-local kernel
        sa, sb = datagen.scale_pair(seed=3)
        c_slice = torch.from_numpy(o.scale_cast(acc, float(sa), float(sb), o.OUT_F32))
        slabs = sharding.all_gather_slabs(c_slice)
        assert tuple(slabs.shape) == (world, M, N // world)
        full = sharding.slabs_to_matrix(slabs)
        ref = o.scale_cast(o.gemm_i8(a, b_full, True), float(sa), float(sb), o.OUT_F32)
        ok = np.array_equal(full.numpy(), ref)
        # max-over-ranks timing reduction as the benchmark does it
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok = ok and t.item() == float(world)
        open(os.path.join(out_dir, f"rank{rank}.ok" if ok else f"rank{rank}.bad"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_column_shards_gather_to_the_full_product(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, 24, 64, 48, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["rank0.ok", "rank1.ok"]
