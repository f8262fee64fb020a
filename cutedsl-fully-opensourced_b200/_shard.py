"""How rows and experts are split over the ranks of a job (pure Python: no torch, no CUDA library)."""
from __future__ import annotations

from typing import Tuple


def shard_rows(rows: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """Contiguous row block of ``rank``: (start, count).  Blocks are multiples of ``multiple`` (so that a rank owns
    whole 128x4 scale-factor tiles) except that the last ranks may get fewer (or zero) rows when ``rows`` runs out."""
    if world < 1 or not 0 <= rank < world or rows < 0:
        raise ValueError("bad rows / world / rank")
    units = -(-rows // multiple)
    per, extra = divmod(units, world)
    start_u = rank * per + min(rank, extra)
    count_u = per + (1 if rank < extra else 0)
    start = min(rows, start_u * multiple)
    end = min(rows, (start_u + count_u) * multiple)
    return start, end - start


def shard_experts(num_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous expert range of ``rank``: (first expert, number of local experts)."""
    if num_experts % world != 0:
        raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
    per = num_experts // world
    return rank * per, per
