"""Column-sharded GEMM across the GPUs of one box: C[:, n0:n1] = A x B[:, n0:n1].

The reference has nothing multi-GPU (no NCCL, no cudaSetDevice, every launch on the default
stream, e.g. src/gemm/sm80_gemm_kernel_v4.cu:344-349); this is the sharding the large int8
configuration asks for. One process per GPU. A is replicated, rank r owns a contiguous block of
B's columns and computes the matching block of C with the ordinary single-GPU kernel -- there is
no inter-GPU traffic inside the GEMM and therefore no data-path collective. Assembling C is an
optional, separately timed all-gather (NCCL on GPUs, any torch.distributed backend in tests) -- or
no separate step at all: with :class:`GatheredOutput` every rank's GEMM epilogue stores its tiles
into the matching column block of *every* rank's full matrix (stores over NVLink to buffers mapped
from the other processes), so the gathered row-major C exists on all GPUs when the GEMMs end.

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


class GatheredOutput:
    """A full row-major C [M, n_total] on every rank, each mapped into every other rank's process.

    Collective over ``group`` (any backend; only small pickled objects are exchanged): every rank allocates its
    matrix, exports the allocation, and maps the others'. ``dst_ptrs(n0)`` then gives, for this rank's column
    block starting at ``n0``, the address of that block in every rank's matrix -- this rank's own first.
    The buffers are written by stores only; nothing is ever loaded from another GPU.
    """

    def __init__(self, M: int, n_total: int, dtype, device, group=None):
        import torch
        import torch.distributed as dist
        from . import peer_export, peer_open, peer_tensor
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.M, self.n_total = int(M), int(n_total)
        # a device allocation of its own (not a piece of torch's caching allocator, whose blocks hold unrelated
        # tensors): the exported handle covers the whole allocation that contains the matrix
        self.local, self._block = peer_tensor((self.M, self.n_total), dtype, self.device)
        handle, offset = peer_export(self.local)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, (handle, offset), group=group)
        self._opened = []
        self.base_ptrs = []
        for r, (h, off) in enumerate(everyone):
            if r == self.rank:
                self.base_ptrs.append(self.local.data_ptr())
            else:
                base = peer_open(h, self.device)
                self._opened.append(base)
                self.base_ptrs.append(base + off)

    @property
    def ldc(self) -> int:
        return self.local.stride(0)

    def dst_ptrs(self, n0: int) -> List[int]:
        """Addresses of column ``n0`` of row 0 in every rank's matrix, this rank's own first."""
        off = int(n0) * self.local.element_size()
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.base_ptrs[r] + off for r in order]

    def close(self) -> None:
        """Collective: unmaps the other ranks' matrices, after everyone has finished with them."""
        import torch
        import torch.distributed as dist
        from . import peer_close
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for base in self._opened:
            peer_close(base, self.device)
        self._opened = []
        dist.barrier(group=self.group)  # nobody maps this rank's matrix any more
        self.local = None
        self._block.free()


def sharded_mix_gemm_gather(a, b_slice, scale_a, scale_b, out: GatheredOutput) -> None:
    """Rank-local GEMM of the column-sharded product whose epilogue writes this rank's column block into every
    rank's full matrix: out[:, n0:n1] = cast(sa*sb*(a x b_slice^T)) on all GPUs (K-major B slice [n_per, K]).
    Enqueues only; synchronise the device and let the ranks meet (a barrier) before reading ``out.local``."""
    from . import gemm_multi_dst
    n_per = b_slice.shape[0]
    n0, n1 = partition_columns(out.n_total, out.world, out.rank)
    if n1 - n0 != n_per:
        raise ValueError(f"B slice has {n_per} rows, this rank owns {n1 - n0} columns")
    gemm_multi_dst(a, b_slice, scale_a, scale_b, out.dst_ptrs(n0), out.ldc, out.local.dtype, n_per, b_kmajor=True)
