"""The allocation-free GEMM entry point against the allocating one, through the C ABI.

``fk_gemm_bf16_host_noalloc`` is for callers that cannot call the CUDA allocator from the call
(latency-bound serving loops, processes whose device memory belongs to another pool): it stages
A, B and C in an array that is part of the library. Both entry points run the same kernel, so
their outputs must be equal bit for bit. Two calls in a row, of different shapes, check that what
the shared array keeps from one call does not leak into the next. This file sorts last so that a
run stopping at the first failure has already run every other test.
"""
import numpy as np
import pytest

import oracle
from ferro_kittens_b200 import FerroKittensError, gemm
from ferro_kittens_b200._lib import FK_ERR_SHAPE, FK_ERR_TOO_LARGE

pytestmark = pytest.mark.gpu


def _operands(m, n, k, seed):
    rng = np.random.default_rng(seed)
    # bf16 words of N(0, 1) values: the top 16 bits of the fp32 pattern.
    a = (rng.standard_normal((m, k)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    b = (rng.standard_normal((n, k)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    return a, b


def test_two_calls_in_a_row_match_the_allocating_entry_point(device):
    for seed, (m, n, k) in enumerate([(1024, 768, 512), (512, 256, 1024)]):
        a, b = _operands(m, n, k, seed)
        expected = np.zeros((m, n), dtype=np.uint16)
        got = np.full((m, n), 0xFFFF, dtype=np.uint16)
        gemm.run_host(a, b, expected, m, n, k)
        gemm.run_host_noalloc(a, b, got, m, n, k)
        assert np.array_equal(got, expected), f"call {seed}: {(got != expected).sum()} words differ"


def test_the_references_exact_gate_through_this_entry_point(device):
    """Not only equal to its sibling: the reference's own integer operands and exact check
    (examples/src/gemm.rs:434-440, 544-578), twice in a row at two shapes."""
    for m, n, k in [(512, 256, 256), (1024, 1280, 320)]:
        a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
        got = np.full((m, n), 0xFFFF, dtype=np.uint16)
        gemm.run_host_noalloc(a, b, got, m, n, k)
        assert oracle.gemm_check_c(got, m, n, k)[0] == 0


def test_a_shape_the_tiling_does_not_divide_is_refused_before_anything_is_copied(device):
    a = np.zeros((128, 64), dtype=np.uint16)
    b = np.zeros((256, 64), dtype=np.uint16)
    c = np.full((128, 256), 0x1234, dtype=np.uint16)
    with pytest.raises(FerroKittensError, match="does not divide the 256x256x64 tiling") as error:
        gemm.run_host_noalloc(a, b, c, 128, 256, 64)
    assert error.value.code == FK_ERR_SHAPE
    assert (c == 0x1234).all()
    with pytest.raises(FerroKittensError, match="group width of 0") as error:
        gemm.run_host_noalloc(np.zeros((256, 64), dtype=np.uint16), b, np.zeros((256, 256), dtype=np.uint16),
                              256, 256, 64, group=0)
    assert error.value.code == FK_ERR_SHAPE
    # a traversal width past anything sensible is clamped, not overflowed
    m, n, k = 512, 512, 128
    a, b = oracle.gemm_stage("a", m, k), oracle.gemm_stage("b", n, k)
    got = np.zeros((m, n), dtype=np.uint16)
    gemm.run_host_noalloc(a, b, got, m, n, k, group=0xFFFFFFFF)
    assert oracle.gemm_check_c(got, m, n, k)[0] == 0


def test_shapes_past_the_built_in_staging_are_refused(device):
    m, n, k = 2048, 2048, 4096  # A is 16 MiB
    a = np.zeros((m, k), dtype=np.uint16)
    b = np.zeros((n, k), dtype=np.uint16)
    c = np.zeros((m, n), dtype=np.uint16)
    with pytest.raises(FerroKittensError, match="built-in staging holds 8388608 bytes") as error:
        gemm.run_host_noalloc(a, b, c, m, n, k)
    assert error.value.code == FK_ERR_TOO_LARGE
