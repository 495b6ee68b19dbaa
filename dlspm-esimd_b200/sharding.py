"""Work distribution for one process per GPU (torch.distributed ranks).

Two cases, as the workloads shard:
  * a batch of independent SpMMs: every rank computes the same longest-processing-time assignment
    from the problem weights nnz*N and keeps its own problems; no data moves between ranks;
  * one large SpMM: rows are cut into blocks of about nnz/world nonzeros, every rank computes its
    block of C, and the blocks are gathered (the one exchange step of the path).
The partitioners are the C functions of the library (dlspm_partition_*_host), so the C++ drivers and
these ranks agree on the assignment.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np


def my_problems(pkg, weights: np.ndarray, rank: int, world: int) -> np.ndarray:
    """Indices (ascending) of the problems owned by `rank` under the LPT assignment."""
    owner = pkg.partition_lpt(np.asarray(weights, dtype=np.float64), world)
    return np.nonzero(owner == rank)[0]


def row_block(pkg, row_offsets: np.ndarray, rank: int, world: int):
    """(first_row, last_row_exclusive, bounds) of the row block of `rank`."""
    bounds = pkg.partition_rows_by_nnz(np.ascontiguousarray(row_offsets, dtype=np.int32), world)
    return int(bounds[rank]), int(bounds[rank + 1]), bounds


def rebase_offsets(row_offsets: np.ndarray, r0: int, r1: int) -> np.ndarray:
    """Offsets of rows r0..r1-1 relative to the block's first nonzero (column indices stay as they are)."""
    return (row_offsets[r0:r1 + 1] - row_offsets[r0]).astype(np.int32)


def gather_row_blocks(c_local, bounds: Sequence[int], N: int, group=None):
    """All-gathers the C row blocks of all ranks into one (M x N) tensor on every rank.

    Blocks have different heights, so every rank contributes a block padded to the tallest one and
    the padding is dropped after the collective (one all_gather_into_tensor, NCCL on GPUs).
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    heights = [int(bounds[r + 1] - bounds[r]) for r in range(world)]
    tallest = max(heights)
    padded = c_local.new_zeros((tallest, N))
    padded[: c_local.shape[0]] = c_local
    out = c_local.new_empty((world * tallest, N))
    dist.all_gather_into_tensor(out, padded, group=group)
    parts: List = [out[r * tallest: r * tallest + heights[r]] for r in range(world)]
    return torch.cat(parts, dim=0)
