"""How one GEMM is split over the GPUs of a box: one process per GPU, no data-path collective
unless K is split.

The reference is single-GPU (cudaSetDevice(0), matmul_shmem_tc_async_opt_port_2.cu:1503-1510);
output tiles are independent, so the split is by rows of A (and D), by rows of B^T (columns of D),
or by K with an fp32 reduce-scatter of the partial products.
"""
from __future__ import annotations

from dataclasses import dataclass


def _split(total: int, world: int, rank: int, align: int) -> tuple[int, int]:
    """Contiguous range of `total` for `rank`, boundaries on multiples of `align` (the last range
    takes what is left). Ranges cover [0, total) without overlap; a range may be empty."""
    if world < 1 or not (0 <= rank < world) or align < 1 or total < 0:
        raise ValueError("bad split arguments")
    units = (total + align - 1) // align
    lo = (units * rank) // world
    hi = (units * (rank + 1)) // world
    return min(lo * align, total), min(hi * align, total)


@dataclass(frozen=True)
class Shard:
    kind: str      # "m", "n" or "k"
    rank: int
    world: int
    begin: int
    end: int

    @property
    def size(self) -> int:
        return self.end - self.begin


def m_shard(M: int, world: int, rank: int, tile_m: int = 128) -> Shard:
    """Rows [begin, end) of A and D for this rank; B^T is replicated; no collective."""
    b, e = _split(M, world, rank, tile_m)
    return Shard("m", rank, world, b, e)


def n_shard(N: int, world: int, rank: int, tile_n: int = 256) -> Shard:
    """Rows [begin, end) of B^T (= columns of D) for this rank; A is replicated; the column
    blocks of D stay distributed; no collective."""
    b, e = _split(N, world, rank, tile_n)
    return Shard("n", rank, world, b, e)


def k_shard(K: int, world: int, rank: int, segment_dim_k: int = 64) -> Shard:
    """Columns [begin, end) of A and of B^T for this rank; every rank produces a full m x n fp32
    partial, combined by reduce_scatter_rows."""
    b, e = _split(K, world, rank, segment_dim_k)
    return Shard("k", rank, world, b, e)


def reduce_scatter_rows(partial, group=None):
    """Sum of the ranks' partial m x n products, scattered by rows: rank r keeps rows
    [r*m/world, (r+1)*m/world). One torch.distributed reduce-scatter (NCCL over NVLink on GPUs,
    gloo on CPU). m must be a multiple of the world size."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    m, n = partial.shape
    if m % world:
        raise ValueError("rows must divide by the world size")
    out = torch.empty((m // world, n), dtype=partial.dtype, device=partial.device)
    if world == 1:
        out.copy_(partial)
        return out
    if partial.is_cuda:
        dist.reduce_scatter_tensor(out, partial.contiguous(), op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce_scatter: all-reduce, then keep the owned rows
        full = partial.clone()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        r = dist.get_rank(group)
        out.copy_(full[r * (m // world):(r + 1) * (m // world)])
    return out
