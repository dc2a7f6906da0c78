"""Partition of the op batch over ranks.

Every (batch, head) row of the memory path is an independent scan with its own archive
(the reference indexes the archive within a batch row: grm/csrc/batched_gather.cu:38-41), so a
job over ``world`` GPUs gives rank ``r`` a contiguous slice of rows and nothing is exchanged on
the data path.  ``gather_rows`` exists for verification only.
"""

from __future__ import annotations

from typing import List, Tuple


def row_range(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open row interval of ``rank``: sizes differ by at most one, earlier ranks get the extras."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n_rows < 0:
        raise ValueError("n_rows must be non-negative")
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def all_row_ranges(n_rows: int, world: int) -> List[Tuple[int, int]]:
    return [row_range(n_rows, r, world) for r in range(world)]


def shard_rows(tensor, rank: int, world: int):
    """View of the rows of ``tensor`` (dim 0) owned by ``rank``."""
    start, stop = row_range(tensor.shape[0], rank, world)
    return tensor[start:stop]


def gather_rows(local, n_rows: int, group=None):
    """All ranks' row slices concatenated in rank order (verification only: one all_gather).

    Works with any ``torch.distributed`` backend; slices may have different lengths.
    """
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ranges = all_row_ranges(n_rows, world)
    longest = max(stop - start for start, stop in ranges)
    padded = local.new_zeros((longest,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    return torch.cat([piece[: stop - start] for piece, (start, stop) in zip(pieces, ranges)], dim=0)
