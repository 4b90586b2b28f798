"""The multi-GPU split on the CPU: shard arithmetic, and a world-size-2 gloo run in which each
rank computes its own block with the oracle and the blocks tile the whole, with no collective on
the data path (the gather below is the test's own check)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from ferro_kittens_b200 import shard


def test_gemm_columns_tile_the_matrix_in_whole_tiles():
    for n, world in [(16384, 1), (16384, 2), (16384, 4), (16384, 8), (28672, 8), (768, 2), (1280, 4)]:
        blocks = [shard.gemm_columns(n, world, rank) for rank in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert all(start % 256 == 0 and stop % 256 == 0 for start, stop in blocks)
        sizes = [stop - start for start, stop in blocks]
        assert max(sizes) - min(sizes) <= 256
    with pytest.raises(ValueError):
        shard.gemm_columns(1000, 2, 0)
    with pytest.raises(ValueError):
        shard.gemm_columns(1024, 2, 2)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 6, 8])
def test_gemm_blocks_tile_c_and_upload_least(world):
    """Host-resident operands: the grid of C blocks covers C once, in whole tiles, and no other
    whole-tile grid uploads fewer operand rows per rank."""
    m = n = 16384
    rows, columns = shard.gemm_grid(m, n, world)
    assert rows * columns == world
    covered = np.zeros((m // 256, n // 256), dtype=np.int32)
    for rank in range(world):
        r0, r1, c0, c1 = shard.gemm_block(m, n, world, rank)
        assert r0 % 256 == 0 and r1 % 256 == 0 and c0 % 256 == 0 and c1 % 256 == 0
        covered[r0 // 256:r1 // 256, c0 // 256:c1 // 256] += 1
    assert (covered == 1).all()
    for other in range(1, world + 1):
        if world % other == 0 and m % (256 * other) == 0 and n % (256 * (world // other)) == 0:
            assert m / rows + n / columns <= m / other + n / (world // other)
    assert shard.gemm_grid(m, n, 8) == (2, 4) and shard.gemm_grid(m, n, 2) == (1, 2)


@pytest.mark.parametrize("m, world, blocks", [(16384, 8, 4), (16384, 2, 4), (16384, 1, 16), (8192, 4, 3), (1024, 2, 8),
                                              (512, 2, 4), (1536, 3, 2)])
def test_gathered_row_blocks_cover_a_once(m, world, blocks):
    """A replicated by all-gather: the ranks' shares tile A, the blocks tile a share in whole 256-row
    tiles, and every row of A appears in exactly one row of exactly one gathered buffer."""
    shares = [shard.a_rows(m, world, rank) for rank in range(world)]
    assert shares[0][0] == 0 and shares[-1][1] == m
    assert all(a[1] == b[0] for a, b in zip(shares, shares[1:]))
    assert len({stop - start for start, stop in shares}) == 1
    plan = shard.gather_blocks(m, world, blocks)
    assert 1 <= len(plan) <= blocks
    assert plan[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(plan, plan[1:]))
    assert plan[-1][0] + plan[-1][1] == m // world and all(rows % 256 == 0 and rows > 0 for _, rows in plan)
    seen = np.zeros(m, dtype=np.int32)
    for offset, rows in plan:
        for buffer_row in range(world * rows):
            seen[shard.gathered_row(m, world, offset, rows, buffer_row)] += 1
    assert (seen == 1).all()


def test_a_rows_refuses_unequal_shares():
    with pytest.raises(ValueError):
        shard.a_rows(768, 2, 0)  # 1.5 tiles each
    with pytest.raises(ValueError):
        shard.a_rows(1024, 2, 2)


def test_planes_tile_the_batch():
    for total, world in [(256, 8), (128, 8), (6, 4), (1, 2)]:
        blocks = [shard.planes(total, world, rank) for rank in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))


def test_row_tiles_never_split_a_tile():
    for rows, world in [(4 * 1024 * 1024, 8), (128 * 7, 4), (128, 2), (128 * 149, 8)]:
        blocks = [shard.row_tiles(rows, world, rank) for rank in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == rows
        assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
        assert all(start % 128 == 0 and stop % 128 == 0 for start, stop in blocks)
    with pytest.raises(ValueError):
        shard.row_tiles(130, 2, 0)


def _free_port() -> int:
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 256, 768, 128
        a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
        start, stop = shard.gemm_columns(n, world, rank)
        block, _ = oracle.gemm_rows(a, b[start:stop], 0, m)
        # timing aggregation as the benchmark does it: the slowest rank sets the step time
        seconds = torch.tensor([0.25 + rank], dtype=torch.float64)
        dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
        gathered = [None] * world
        dist.all_gather_object(gathered, (start, stop, block.tobytes()))
        if rank == 0:
            whole = np.zeros((m, n), dtype=np.uint16)
            for s, e, raw in gathered:
                whole[:, s:e] = np.frombuffer(raw, dtype=np.uint16).reshape(m, e - s)
            results.put((oracle.gemm_check_c(whole, m, n, k)[0], float(seconds.item())))
    finally:
        dist.destroy_process_group()


def _gather_worker(rank: int, world: int, port: int, results):
    """The host-buffer pipeline's bookkeeping with gloo standing in for NCCL and the oracle for
    the kernel: each rank holds only its share of A, the blocks are all-gathered, the GEMM of a
    gathered buffer lands in the rows `gathered_row` names."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k = 1024, 512, 128
        a_whole, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
        row0, row1 = shard.a_rows(m, world, rank)
        a_share = torch.from_numpy(a_whole[row0:row1].astype(np.int32))  # this rank never touches the rest
        start, stop = shard.gemm_columns(n, world, rank)
        c_block = np.zeros((m, stop - start), dtype=np.uint16)
        for offset, rows in shard.gather_blocks(m, world, 2):
            gathered = torch.empty((world * rows, k), dtype=torch.int32)
            dist.all_gather_into_tensor(gathered, a_share[offset:offset + rows].contiguous())
            product, _ = oracle.gemm_rows(gathered.numpy().astype(np.uint16), b[start:stop], 0, world * rows)
            for buffer_row in range(world * rows):
                c_block[shard.gathered_row(m, world, offset, rows, buffer_row)] = product[buffer_row]
        pieces = [None] * world
        dist.all_gather_object(pieces, (start, stop, c_block.tobytes()))
        if rank == 0:
            whole = np.zeros((m, n), dtype=np.uint16)
            for s, e, raw in pieces:
                whole[:, s:e] = np.frombuffer(raw, dtype=np.uint16).reshape(m, e - s)
            results.put(oracle.gemm_check_c(whole, m, n, k)[0])
    finally:
        dist.destroy_process_group()


def test_two_ranks_complete_a_by_all_gather_and_tile_c():
    context = mp.get_context("spawn")
    results = context.Queue()
    world, port = 2, _free_port()
    workers = [context.Process(target=_gather_worker, args=(rank, world, port, results)) for rank in range(world)]
    for worker in workers:
        worker.start()
    wrong = results.get(timeout=120)
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    assert wrong == 0


def test_two_ranks_compute_disjoint_blocks_that_tile_c():
    context = mp.get_context("spawn")
    results = context.Queue()
    world, port = 2, _free_port()
    workers = [context.Process(target=_worker, args=(rank, world, port, results)) for rank in range(world)]
    for worker in workers:
        worker.start()
    wrong, slowest = results.get(timeout=120)
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    assert wrong == 0
    assert slowest == 1.25
