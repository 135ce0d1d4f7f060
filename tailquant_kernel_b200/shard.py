"""Token-row sharding of the split linear across the GPUs of one box.

Every stage of the path is independent per token row (rotation, select, quantisation, the GEMM row,
the tail row), so M rows are cut into contiguous slabs, one per rank, prepared weights are replicated,
and no collective is needed on the data path.  The reference has no distributed code at all; it uses
its eight GPUs as eight independent job slots (run_qwen3_8b_v2_ratio_split_latency_v56.sh:87-121).
"""
from __future__ import annotations

from typing import List, Tuple


def row_shard(M: int, rank: int, world: int) -> Tuple[int, int]:
    """(first row, row count) of `rank`: contiguous, sizes differ by at most one, earlier ranks
    take the extra rows."""
    if world < 1 or not (0 <= rank < world) or M < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(M, world)
    start = rank * base + min(rank, extra)
    return start, base + (1 if rank < extra else 0)


def all_shards(M: int, world: int) -> List[Tuple[int, int]]:
    return [row_shard(M, r, world) for r in range(world)]


def column_shard(N: int, rank: int, world: int, multiple: int = 64) -> Tuple[int, int]:
    """(first column, column count) of an optional column-parallel split of a wide projection
    (its outputs are all-gathered afterwards); slabs are multiples of `multiple` columns."""
    if N % multiple:
        raise ValueError("N must be a multiple of the slab granularity")
    s, c = row_shard(N // multiple, rank, world)
    return s * multiple, c * multiple
