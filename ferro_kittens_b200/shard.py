"""How the two paths split across the GPUs of one node: independent shards,
no collective on the data path.

The GEMM replicates A and gives each rank a contiguous block of B's rows (C's
columns); attention (forward and backward) gives each rank a contiguous range of
(batch x head) planes; the row kernels give each rank a contiguous range of whole
128-row tiles.
"""
from __future__ import annotations

from .gemm import BLOCK_N


def gemm_columns(n: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the C columns (rows of the K-major B) rank ``rank`` owns.

    Blocks are whole 256-column tiles; the first ``tiles % world`` ranks take one extra.
    """
    if n % BLOCK_N:
        raise ValueError(f"{n} columns is not a whole number of {BLOCK_N}-column tiles")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    tiles = n // BLOCK_N
    base, extra = divmod(tiles, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * BLOCK_N, stop * BLOCK_N


def planes(total: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the attention planes rank ``rank`` owns."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def row_tiles(rows: int, world: int, rank: int, tile: int = 128) -> tuple[int, int]:
    """[start, stop) of the rows rank ``rank`` owns, in whole ``tile``-row tiles (the unit the
    whole-tile statistic is taken over, so no tile is ever split between GPUs)."""
    if rows % tile:
        raise ValueError(f"{rows} rows is not a whole number of {tile}-row tiles")
    start, stop = planes(rows // tile, world, rank)
    return start * tile, stop * tile
