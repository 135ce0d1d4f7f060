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


def gather_columns(y_local, N: int, group=None, multiple: int = 64):
    """The one exchange step of the column-parallel split: every rank holds the [M, n_r] output slab of its
    channels (`column_shard`) and receives the full [M, N] output.  One `all_gather_into_tensor` over the process
    group (NCCL over NVLink on GPUs, gloo on CPU) into a [world, M, widest] buffer, then ONE strided copy into the
    [M, N] result when the slabs are equal (N / multiple divisible by the world size: every projection of the
    benchmarked models), or one copy per rank when a narrower last slab was padded to the widest."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = [column_shard(N, r, world, multiple) for r in range(world)]
    M = y_local.shape[0]
    if y_local.shape[1] != shards[rank][1]:
        raise RuntimeError(f"rank {rank} holds {y_local.shape[1]} columns, its shard has {shards[rank][1]}")
    widest = max(c for _, c in shards)
    equal = all(c == widest for _, c in shards)
    send = y_local.contiguous()
    if not equal and send.shape[1] != widest:
        send = torch.zeros((M, widest), dtype=y_local.dtype, device=y_local.device)
        send[:, : y_local.shape[1]] = y_local
    flat = torch.empty((world * M, widest), dtype=y_local.dtype, device=y_local.device)  # rank-major concatenation
    dist.all_gather_into_tensor(flat, send, group=group)
    buf = flat.view(world, M, widest)
    out = torch.empty((M, N), dtype=y_local.dtype, device=y_local.device)
    if equal:
        out.view(M, world, widest).copy_(buf.permute(1, 0, 2))
    else:
        for r, (s0, c) in enumerate(shards):
            out[:, s0:s0 + c] = buf[r, :, :c]
    return out


class ColumnParallelSplitLinear:
    """Optional N-split of one wide projection (e.g. gate_up): each rank prepares and runs the split linear on
    its slab of output channels and the outputs are all-gathered.  Token-row sharding (no collective) stays the
    default; this trades one exchange of M x N bf16 for 1/world of the weight traffic per GPU."""

    def __init__(self, weight, rank: int, world: int, bias=None, group=None, multiple: int = 64, **kw):
        from .linear import SplitLinear
        self.N = int(weight.shape[0])
        self.group, self.multiple = group, multiple
        s0, c = column_shard(self.N, rank, world, multiple)
        self.local = SplitLinear(weight[s0:s0 + c].contiguous(), bias=None if bias is None else bias[s0:s0 + c], **kw)

    def forward(self, x):
        y = self.local(x)
        lead = y.shape[:-1]
        full = gather_columns(y.reshape(-1, y.shape[-1]), self.N, self.group, self.multiple)
        return full.view(*lead, self.N)

    __call__ = forward
