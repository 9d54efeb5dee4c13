"""Row sharding of a projection across the GPUs of one node.

y = W x is a set of independent dot products, one per output row, so a tensor is split by
output rows: rank r of `world` owns rows [r*n/world, (r+1)*n/world) and the full output is the
concatenation of the ranks' pieces in rank order (an all-gather). Matrices with too few rows to
be worth a collective, or whose row count does not divide evenly, stay replicated on every rank.
"""
from __future__ import annotations

SHARD_MIN_ROWS = 4096


def is_sharded(n_rows: int, world: int, min_rows: int = SHARD_MIN_ROWS) -> bool:
    return world > 1 and n_rows >= min_rows and n_rows % world == 0


def row_range(n_rows: int, rank: int, world: int, min_rows: int = SHARD_MIN_ROWS) -> tuple[int, int]:
    """Rows of an n_rows-row tensor that `rank` computes: its shard, or all rows when the tensor is replicated."""
    if not 0 <= rank < max(world, 1):
        raise ValueError("rank out of range")
    if not is_sharded(n_rows, world, min_rows):
        return 0, n_rows
    per = n_rows // world
    return rank * per, (rank + 1) * per
