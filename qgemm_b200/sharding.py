"""Column-sharded GEMM across the GPUs of one box: C[:, n0:n1] = A x B[:, n0:n1].

The reference has nothing multi-GPU (no NCCL, no cudaSetDevice, every launch on the default
stream, e.g. src/gemm/sm80_gemm_kernel_v4.cu:344-349); this is the sharding the large int8
configuration asks for. One process per GPU. A is replicated, rank r owns a contiguous block of
B's columns and computes the matching block of C with the ordinary single-GPU kernel -- there is
no inter-GPU traffic inside the GEMM and therefore no data-path collective. Assembling C is an
optional, separately timed all-gather (NCCL on GPUs, any torch.distributed backend in tests).

Gathered layout: NCCL concatenates along the slowest dimension while column blocks of a row-major
C are strided, so the gather produces *slabs* ``[world][M][n_per_rank]`` (zero extra work);
:func:`slabs_to_matrix` turns them into a row-major ``[M, N]`` when a consumer needs that.
"""
from __future__ import annotations

from typing import List, Tuple


def partition_columns(n_total: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open column range [n0, n1) of rank ``rank``. N must divide evenly so that every rank's
    slab has the same shape (what all_gather_into_tensor needs); ragged N is rejected, not padded."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} of world size {world_size}")
    if n_total % world_size != 0:
        raise ValueError(f"N={n_total} is not divisible by the number of ranks {world_size}")
    per = n_total // world_size
    return rank * per, (rank + 1) * per


def all_partitions(n_total: int, world_size: int) -> List[Tuple[int, int]]:
    return [partition_columns(n_total, world_size, r) for r in range(world_size)]


def sharded_mix_gemm(a, b_slice, scale_a, scale_b, c_slice) -> None:
    """Rank-local part: c_slice[M, n_per] = cast(sa*sb*(a[M,K] x b_slice[n_per,K]^T)), K-major B slice."""
    from . import mix_gemm
    mix_gemm(a, b_slice, scale_a, scale_b, c_slice, b_kmajor=True)


def all_gather_slabs(c_slice, group=None):
    """All-gather the per-rank C slices into slabs [world, M, n_per]. Returns the slab tensor."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    M, n_per = c_slice.shape
    out = torch.empty((world, M, n_per), dtype=c_slice.dtype, device=c_slice.device)
    if not c_slice.is_contiguous():
        c_slice = c_slice.contiguous()
    dist.all_gather_into_tensor(out.view(world * M, n_per), c_slice, group=group)
    return out


def slabs_to_matrix(slabs):
    """[world, M, n_per] slabs -> row-major [M, world*n_per]."""
    world, M, n_per = slabs.shape
    return slabs.permute(1, 0, 2).reshape(M, world * n_per)
