"""Row sharding of a population over the ranks of one `torch.distributed` process group.

The reference keeps the whole state on every rank and only splits the evaluation
(evox/workflows/std_workflow.py:167-189). Here the state itself is split: rank r owns the
contiguous block of rows `torch.tensor_split` would give it, and the only data that crosses
ranks each generation is one best-particle record per rank.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """[start, end) of rank's rows; identical to `Tensor.tensor_split(world_size)[rank]`
    (the first `n_rows % world_size` shards get one extra row)."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of size {world_size}")
    base, extra = divmod(n_rows, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def group_info(group=None) -> tuple[int, int]:
    """(rank, world_size) of `group`, or (0, 1) when torch.distributed is not initialised."""
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def allgather_records(record: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Concatenate every rank's 1-D record in rank order (one small allgather). `out`, when given,
    receives the result (world_size * record.numel() elements) instead of a fresh tensor."""
    rank, world = group_info(group)
    if world == 1:
        return record
    if out is None:
        out = torch.empty(world * record.numel(), dtype=record.dtype, device=record.device)
    dist.all_gather_into_tensor(out.view(-1), record, group=group)
    return out
