"""The counter-based operand generator: a value depends on (seed, tensor, index) only, so a
shard generated on its own equals the same rows of the whole, on any device."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from ferro_kittens_b200 import seeded

MASK = (1 << 64) - 1


def _mix64(x: int) -> int:
    z = (x + 0x9E3779B97F4A7C15) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def _word(seed, tensor, index, draw):
    key = (seed * 0xD1342543DE82EF95 + tensor * 0xA0761D6478BD642F + draw * 0xE7037ED1A0B428DB) & MASK
    return _mix64(_mix64(index) ^ key)


def test_mix64_matches_plain_integer_arithmetic():
    values = [0, 1, 2, 12345, (1 << 63) - 1, 1 << 40]
    got = seeded.mix64(torch.tensor(values, dtype=torch.int64)).numpy().view(np.uint64)
    assert [int(v) for v in got] == [_mix64(v) for v in values]


def test_uniform_and_normal_follow_their_definitions():
    for index in (0, 7, 1_000_003):
        u = seeded.uniform(3, 1, index, 1)[0].item()
        assert u == np.float32((_word(3, 1, index, 0) >> 40) * (2.0 / (1 << 24))) - np.float32(1.0)
        lanes = sum((_word(3, 1, index, 1 + d) >> (16 * lane)) & 0xFFFF for d in range(3) for lane in range(4))
        assert seeded.normal(3, 1, index, 1)[0].item() == (lanes - 12 * 32767.5) / 65536.0


def test_a_shard_generated_alone_equals_the_same_rows_of_the_whole():
    whole = seeded.bf16_rows("normal", 2, 1, 0, 96, 64, 0.02, chunk_rows=40)
    for row0, rows in ((0, 10), (17, 31), (90, 6)):
        part = seeded.bf16_rows("normal", 2, 1, row0, rows, 64, 0.02, chunk_rows=7)
        assert torch.equal(part, whole[row0:row0 + rows])
    other = seeded.bf16_rows("normal", 2, 0, 0, 96, 64, 0.02)
    assert not torch.equal(other, whole)  # another tensor id, other values


def test_moments_and_ranges():
    n = seeded.normal(1, 0, 0, 1 << 20)
    assert abs(n.mean().item()) < 5e-3 and abs(n.var().item() - 1.0) < 5e-3
    assert n.abs().max().item() <= 6.0
    u = seeded.uniform(0, 0, 0, 1 << 20)
    assert -1.0 <= u.min().item() and u.max().item() < 1.0
    assert abs(u.mean().item()) < 5e-3 and abs(u.var().item() - 1.0 / 3.0) < 5e-3


@pytest.mark.gpu
def test_host_and_device_produce_the_same_words():
    for kind, scale in (("normal", 1.0 / 128.0), ("normal", 0.02), ("uniform", 1.0)):
        host = seeded.bf16_rows(kind, 4, 2, 5, 300, 128, scale)
        device = seeded.bf16_rows(kind, 4, 2, 5, 300, 128, scale, device="cuda")
        assert torch.equal(host, device.cpu())
