"""How the two paths split across the GPUs of one node: independent shards,
no collective on the data path.

The GEMM replicates A and gives each rank a contiguous block of B's rows (C's
columns) when the operands are resident on the device; from host buffers, where the upload
is the cost, it cuts C into a grid of blocks instead (`gemm_grid`); attention (forward and backward) gives each rank a contiguous range of
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


def gemm_grid(m: int, n: int, world: int, tile: int = BLOCK_N) -> tuple[int, int]:
    """(row blocks, column blocks) with rows x columns = world for a GEMM whose operands start in HOST
    memory: rank (i, j) uploads rows block i of A and rows block j of the K-major B, so the split that
    uploads the fewest bytes per rank minimises m / rows + n / columns. Only splits into whole
    ``tile``-sized blocks count; ties go to fewer row blocks; (1, world) if nothing else divides."""
    best = (1, world)
    cost = None
    for row_blocks in range(1, world + 1):
        if world % row_blocks:
            continue
        column_blocks = world // row_blocks
        if m % (tile * row_blocks) or n % (tile * column_blocks):
            continue
        here = m / row_blocks + n / column_blocks
        if cost is None or here < cost:
            best, cost = (row_blocks, column_blocks), here
    return best


def gemm_block(m: int, n: int, world: int, rank: int) -> tuple[int, int, int, int]:
    """[row0, row1) x [column0, column1) of C that rank ``rank`` owns under :func:`gemm_grid`
    (row-major over the grid: rank = i * column blocks + j)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    row_blocks, column_blocks = gemm_grid(m, n, world)
    if row_blocks == 1:
        column0, column1 = gemm_columns(n, world, rank)
        return 0, m, column0, column1
    i, j = divmod(rank, column_blocks)
    rows, columns = m // row_blocks, n // column_blocks
    return i * rows, (i + 1) * rows, j * columns, (j + 1) * columns


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
