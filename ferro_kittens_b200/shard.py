"""How the two paths split across the GPUs of one node: independent shards,
no collective on the data path.

The GEMM replicates A and gives each rank a contiguous block of B's rows (C's
columns). When the operands start in HOST memory the replication is not paid for over
PCIe: every rank uploads only its own share of A's rows (`a_rows`) and the ranks complete A
in their own HBM over NVLink, block of rows by block of rows (`gather_blocks`), each block's
GEMM starting as soon as it is whole -- staging, outside the kernels, which still read only
their own GPU's memory. Attention (forward and backward) gives each rank a contiguous range
of (batch x head) planes; the row kernels give each rank a contiguous range of whole 128-row
tiles. `gemm_grid` / `gemm_block` describe the alternative of cutting C into a grid of blocks.
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


def a_rows(m: int, world: int, rank: int, tile: int = 2 * 128) -> tuple[int, int]:
    """[start, stop) of the rows of A that rank ``rank`` uploads from host memory when A is
    replicated by an all-gather instead of by ``world`` uploads: whole ``tile``-row pair tiles,
    the same count on every rank (an all-gather moves equal shares)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if m % (tile * world):
        raise ValueError(f"{m} rows do not split into {world} equal shares of whole {tile}-row tiles")
    share = m // world
    return rank * share, (rank + 1) * share


def gather_blocks(m: int, world: int, blocks: int, tile: int = 2 * 128) -> list[tuple[int, int]]:
    """The all-gather schedule of a replicated A: ``[(offset, rows), ...]`` inside every rank's
    share, at most ``blocks`` of them, each whole ``tile``-row tiles. Gathering block ``(offset,
    rows)`` yields a ``[world, rows, k]`` buffer whose slab ``r`` is rows ``[r * share + offset,
    r * share + offset + rows)`` of A -- and, after the GEMM over the buffer, of C."""
    share = a_rows(m, world, 0, tile)[1]
    tiles = share // tile
    count = max(1, min(blocks, tiles))
    base, extra = divmod(tiles, count)
    out, offset = [], 0
    for index in range(count):
        rows = (base + (1 if index < extra else 0)) * tile
        out.append((offset, rows))
        offset += rows
    return out


def gathered_row(m: int, world: int, offset: int, rows: int, buffer_row: int) -> int:
    """Row of A (and of C) that row ``buffer_row`` of the gathered ``[world * rows, k]`` buffer of
    block ``(offset, rows)`` holds."""
    share = m // world
    slab, within = divmod(buffer_row, rows)
    return slab * share + offset + within


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
