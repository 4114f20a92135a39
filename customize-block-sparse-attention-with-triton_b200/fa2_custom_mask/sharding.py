"""Partitioning of the attention work across the GPUs of one box.

Every (batch, head) is independent (own q, k, v and mask slice), so the primary split hands each
rank a contiguous run of the flattened (b, h) index and nothing is exchanged on the data path.
When there are fewer (b, h) units than ranks, the query-block rows of each head are split instead,
balanced by listed-tile count, with that head's K and V replicated on every rank (forward only: a
row split of the backward would need a dK/dV reduction).  The reference's forward grid is one
program per listed (b, h, query block) row (fa2_custom_mask/fa2_custom_mask.py:69-70), so any
subset of rows is a complete launch; the forward entry points take the row range as
`rows=(begin, end)`.
"""
from __future__ import annotations

from bisect import bisect_right
from itertools import accumulate
from typing import List, Sequence, Tuple


def shard_heads(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the flattened (b*H + h) units owned by `rank`; sizes differ by at most 1."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("rank must lie in [0, world_size)")
    base, extra = divmod(n_units, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows_by_tiles(row_tiles: Sequence[int], world_size: int) -> List[Tuple[int, int]]:
    """Splits query-block rows 0..nb-1 into `world_size` contiguous [start, stop) ranges whose
    listed-tile totals are as even as a contiguous split allows: cut k is placed where the
    running total is closest to k/world_size of the whole.  A range may be empty (more ranks than
    rows, or all tiles in a few rows); its rank then has nothing to launch."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    nb = len(row_tiles)
    prefix = [0] + list(accumulate(int(t) for t in row_tiles))  # prefix[r] = tiles of rows < r
    total = prefix[-1]
    bounds = [0]
    for k in range(1, world_size):
        target = total * k / world_size
        r = bisect_right(prefix, target) - 1          # prefix[r] <= target < prefix[r + 1]
        if r < nb and prefix[r + 1] - target < target - prefix[r]:
            r += 1
        bounds.append(min(nb, max(r, bounds[-1])))
    bounds.append(nb)
    return [(bounds[i], bounds[i + 1]) for i in range(world_size)]


def plan(B: int, H: int, world_size: int, rank: int, row_tiles: Sequence[int] | None = None):
    """Returns ("heads", (start, stop)) or, when B*H < world_size and row_tiles is given,
    ("rows", (start, stop)) for the forward row split of every head."""
    units = B * H
    if units >= world_size or row_tiles is None:
        return "heads", shard_heads(units, world_size, rank)
    return "rows", shard_rows_by_tiles(row_tiles, world_size)[rank]
