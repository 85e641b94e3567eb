"""Row-block sharding of a GEMM over one process per GPU.

Every output element depends on one row of A and one column of B, so the
output splits into independent row blocks: rank r owns rows
``[row_begin, row_begin + row_count)`` of A (and its scales), C and D and holds
all of B.  No data moves during the GEMM, and each rank's arithmetic is the
single-GPU arithmetic, so the assembled D is bit-identical to a one-GPU run.
The only collective is an optional all-gather of the D blocks when the caller
wants D replicated (NCCL over NVLink on GPUs; gloo in the CPU tests).

The reference has no multi-device code; this plays the role of its
``partition_gemm`` (gemm/threadblock/threadblock_swizzle.h:47-91) across
devices instead of threads.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional

from . import _capi


@dataclass(frozen=True)
class RowShard:
    rank: int
    world: int
    row_begin: int
    row_count: int


def shard_rows(m: int, world: int, rank: int) -> RowShard:
    """Balanced split of the 128-row tiles of an m-row output (C ABI:
    ``cpuops_b200_shard_rows``)."""
    r0, rn = C.c_int32(0), C.c_int32(0)
    st = _capi.load().cpuops_b200_shard_rows(m, world, rank, C.byref(r0), C.byref(rn))
    if st != 0:
        raise ValueError(f"invalid shard request m={m} world={world} rank={rank}")
    return RowShard(rank, world, r0.value, rn.value)


def shard_plan(m: int, world: int) -> List[RowShard]:
    return [shard_rows(m, world, r) for r in range(world)]


def all_gather_rows(d_local, m: int, group=None):
    """Assemble the replicated row-major D (m x n) from every rank's row block.

    ``d_local`` is this rank's contiguous ``row_count x n`` torch tensor (CPU with
    gloo, CUDA with NCCL).  Blocks may differ in size by one tile, so the gather
    pads to the largest block and trims.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    plan = shard_plan(m, world)
    n = d_local.shape[1]
    max_rows = max(s.row_count for s in plan)
    padded = torch.zeros((max_rows, n), dtype=d_local.dtype, device=d_local.device)
    padded[: d_local.shape[0]] = d_local
    gathered = torch.empty((world, max_rows, n), dtype=d_local.dtype, device=d_local.device)
    dist.all_gather_into_tensor(gathered.view(world * max_rows, n), padded, group=group)
    out = torch.empty((m, n), dtype=d_local.dtype, device=d_local.device)
    for s in plan:
        out[s.row_begin: s.row_begin + s.row_count] = gathered[s.rank, : s.row_count]
    return out
