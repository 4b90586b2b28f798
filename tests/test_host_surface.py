"""Host-side arithmetic and validation behind the C ABI, on the CPU.

Each case restates a host unit test of the reference against this library's
exports: the `grouped` traversal (src/pipeline.rs:182-192, 675-729), swizzle
addresses (src/shared.rs:1966-2056), operand and instruction descriptors
(src/shared.rs:2140-2177, src/mma.rs:572-723), tensor-memory addressing
(src/tmem.rs:487), shared-plan totals (src/plan.rs:320-445), layout shapes and
driver-rule messages (src/global.rs:2089-2225), and that the library exports
every symbol the header declares.
"""
import ctypes
import re
from pathlib import Path

import pytest

from ferro_kittens_b200 import FerroKittensError, _lib
from ferro_kittens_b200._lib import FK_BF16, FK_F32, library
from ferro_kittens_b200.global_layout import GlobalLayout
from ferro_kittens_b200.plan import SharedPlan

ROOT = Path(__file__).resolve().parent.parent
BASE = 0x7F00_0000  # a device address is never dereferenced on the host


def grouped(item, rows, columns, group):
    row, column = ctypes.c_uint32(), ctypes.c_uint32()
    library().fk_grouped(item, rows, columns, group, ctypes.byref(row), ctypes.byref(column))
    return row.value, column.value


# ---------------------------------------------------------------- exports

def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "ferro_kittens.h").read_text()
    declared = set(re.findall(r"\b(fk_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = library()
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


# ---------------------------------------------------------------- traversal

def test_grouped_documented_walk():
    walk = [grouped(item, 4, 3, 2) for item in range(12)]
    assert walk[:4] == [(0, 0), (1, 0), (0, 1), (1, 1)]
    assert len(set(grouped(item, 4, 3, 3) for item in range(12))) == 12


def test_grouped_covers_every_tile_exactly_once():
    for rows in range(1, 18):
        for columns in range(1, 18):
            for group in range(1, 20):
                seen = [grouped(item, rows, columns, group) for item in range(rows * columns)]
                assert all(r < rows and c < columns for r, c in seen)
                assert len(set(seen)) == rows * columns, (rows, columns, group)


def test_grouped_width_one_is_row_major_and_wide_is_column_major():
    for rows in range(1, 10):
        for columns in range(1, 10):
            for item in range(rows * columns):
                assert grouped(item, rows, columns, 1) == (item // columns, item % columns)
                for group in range(rows, rows + 5):
                    assert grouped(item, rows, columns, group) == (item % rows, item // rows)


# ---------------------------------------------------------------- swizzle, descriptors, tmem

def test_swizzled_chunks_fold_the_base_phase_and_permute_each_row():
    lib = library()
    for phase in range(8):
        seen = set()
        for row in range(64):
            for chunk in range(8):
                offset = lib.fk_swizzled_chunk_offset(row, chunk, phase)
                assert offset == row * 128 + ((chunk ^ ((row + phase) & 7)) * 16)
                assert offset // 128 == row
                seen.add(offset // 16)
        assert len(seen) == 64 * 8


def test_operand_descriptor_encodes_like_the_reference():
    lib = library()
    base = 0x4000
    expected = (((base + 32) >> 4) & 0x3FFF) | (1 << 16) | (64 << 32) | (1 << 46) | (2 << 61)
    assert lib.fk_operand_descriptor(base + 32, 16) == expected
    for chunk in range(4):
        k_major = (((base + chunk * 32) >> 4) & 0x3FFF) | (1 << 16) | (64 << 32) | (1 << 46) | (2 << 61)
        mn_major = ((((base + chunk * 2048) >> 4) & 0x3FFF) | (((8192 >> 4) & 0x3FFF) << 16)
                    | (64 << 32) | (1 << 46) | (2 << 61))
        assert lib.fk_operand_descriptor(base + chunk * 32, 16) == k_major
        assert lib.fk_operand_descriptor(base + chunk * 2048, 8192) == mn_major


def test_instruction_descriptor_bit_layout():
    lib = library()

    def spelled(m, n, ta, tb):
        return (1 << 4) | (1 << 7) | (1 << 10) | (int(ta) << 15) | (int(tb) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24)

    for m, n, ta, tb in [(128, 64, 0, 0), (128, 128, 0, 1), (256, 128, 1, 1), (256, 256, 0, 0)]:
        assert lib.fk_instruction_descriptor(m, n, ta, tb) == spelled(m, n, ta, tb)
    orders = {lib.fk_instruction_descriptor(128, 128, a, b) for a in (0, 1) for b in (0, 1)}
    assert len(orders) == 4


def test_tmem_address_is_base_plus_row_shifted_plus_column():
    lib = library()
    assert lib.fk_tmem_address(0x100, 0, 0) == 0x100
    assert lib.fk_tmem_address(0x100, 32, 64) == 0x100 + (32 << 16) + 64


# ---------------------------------------------------------------- plan

def _example_plan():
    plan = SharedPlan.sizing()
    plan.tile_ring(128, 64, 3)
    plan.tile_ring(128, 64, 3)
    plan.semaphores(3)
    plan.semaphores(3)
    plan.semaphore()
    plan.tmem_slot()
    return plan


def test_reference_gemm_plans_are_the_declared_envelopes():
    plan = _example_plan()
    assert plan.bytes() == 98_364
    plan.tile_ring(32, 64, 4)
    assert plan.bytes() == 114_816
    # The experiment walk with the 16-byte-aligned work queue on the end.
    plan = _example_plan()
    plan.reserve(16, 16)
    plan.semaphores(1)
    assert plan.bytes() == 98_392
    plan.tile_ring(32, 64, 4)
    assert plan.bytes() == 114_816


def test_reference_small_kernel_and_flash_plans():
    plan = SharedPlan.sizing()
    plan.tile(128, 128)
    plan.semaphore()
    assert plan.bytes() == 32_776
    plan = SharedPlan.sizing()
    plan.tile(128, 128)
    plan.reserve(4 * 4, SharedPlan.TILE_ALIGN)
    plan.semaphore()
    assert plan.bytes() == 32_792
    plan = SharedPlan.sizing()
    plan.tile(128, 128)
    plan.semaphore()
    plan.reserve(4 * 4, SharedPlan.TILE_ALIGN)
    assert plan.bytes() == 32_912
    flash = SharedPlan.sizing()
    flash.tile(128, 128)
    flash.tile_ring(64, 128, 3)
    flash.tile_ring(64, 128, 3)
    flash.tile(128, 64)
    flash.semaphores(3)
    flash.semaphores(3)
    for _ in range(3):
        flash.semaphore()
    flash.tmem_slot()
    assert flash.bytes() == 147_532


def test_each_reservation_aligns_to_its_own_rule():
    plan = SharedPlan.sizing()
    assert plan.tmem_slot() == 0 and plan.bytes() == 4
    assert plan.tile(8, 64) == 128 and plan.bytes() == 128 + 8 * 64 * 2
    plan = SharedPlan.sizing()
    plan.tmem_slot()
    assert plan.semaphore() == 8 and plan.bytes() == 16
    plan = SharedPlan.sizing()
    plan.reserve(1000, 128)
    assert plan.reserve(24, 16) == 1008 and plan.bytes() == 1008 + 24
    with pytest.raises(ValueError):
        plan.reserve(8, 12)


def test_this_librarys_own_plans_fit_one_cta_per_sm():
    lib = library()
    for total in (lib.fk_gemm_shared_bytes(), lib.fk_flash_shared_bytes()):
        assert 116_736 < total <= 232_448  # admits exactly one CTA per SM
    # gemm: producer, MMA, eight epilogue warps and the item feed.
    # flash: three warpgroups (two softmax teams; loader + MMA), so that registers can move between them.
    assert lib.fk_gemm_threads() == 352 and lib.fk_flash_threads() == 384
    # gemm: 4 stages of two A tiles and one B tile, 8 staging bands, 10 barriers of the operand and
    # accumulator hand-overs, 6 of the item feed, its 16-byte claim answer and two-entry ring, slot, stop word.
    plan = SharedPlan.sizing()
    plan.tile_ring(128, 64, 8)
    plan.tile_ring(128, 64, 4)
    plan.tile_ring(32, 64, 8)
    for count in (4, 4, 1, 1, 2, 2, 1, 1):
        plan.semaphores(count)
    plan.reserve(16, 16)
    plan.reserve(8, 4)
    plan.tmem_slot()
    plan.reserve(4, 4)
    assert plan.bytes() == lib.fk_gemm_shared_bytes()


def test_grid_is_whole_clusters_capped_at_one_per_sm_pair():
    lib = library()
    assert lib.fk_gemm_grid(512, 256, 148) == 4      # one [512, 256] tile, re-cut into two halves
    assert lib.fk_gemm_grid(4096, 4096, 148) == 148
    assert lib.fk_gemm_grid(16384, 16384, 148) == 148
    assert lib.fk_gemm_grid(1024, 512, 148) == 16    # 4 tiles = a short tail: 8 single-half items
    assert lib.fk_gemm_grid(16384, 2048, 148) == 148


def test_traversal_width_follows_the_window_of_items_in_flight():
    lib = library()
    # sqrt(clusters / 2): the fewest operand-panel bytes per wave when a tile row's A panel is twice a tile column's B panel
    from ferro_kittens_b200 import gemm

    assert lib.fk_gemm_group(16384, 16384, 148) == 6 == gemm.GROUP
    assert lib.fk_gemm_group(8192, 28672, 148) == 6
    assert lib.fk_gemm_group(8192, 3584, 148) == 6       # 14 tile columns: wider than the 12.3 the window spans
    assert lib.fk_gemm_group(16384, 2048, 148) == 4      # 8 tile columns: shorter bands
    assert lib.fk_gemm_group(4096, 4096, 132) == 5
    for sm_count in (2, 3, 16, 64, 132, 148, 160):
        for n in (256, 2048, 16384):
            assert 1 <= lib.fk_gemm_group(4096, n, sm_count) <= max(1, sm_count // 2)


def _wave_time(m, n, columns, clusters):
    """Wave-times of [512, 256] items a launch takes with items `columns` wide: whole waves, and a last
    one that costs half when it holds at most half a wave of tiles (it is re-cut into halves)."""
    tiles = -(-m // 512) * (n // columns)
    tail = tiles % clusters
    return (tiles // clusters + (0 if tail == 0 else 0.5 if 2 * tail <= clusters else 1)) * columns / 256


@pytest.mark.parametrize("sm_count", [148, 132, 64])
def test_item_width_follows_the_wave_arithmetic(sm_count):
    lib = library()
    clusters = sm_count // 2
    for m, n, k in [(8192, 3584, 8192), (8192, 7168, 8192), (8192, 14336, 8192), (8192, 28672, 8192),
                    (16384, 16384, 16384), (16384, 2048, 16384), (2048, 5376, 4096), (4096, 10752, 512),
                    (3072, 3072, 4096), (768, 5376, 8192)]:
        chosen = lib.fk_gemm_item_columns(m, n, k, 0, sm_count)
        assert chosen in (256, 224, 192) and n % chosen == 0
        candidates = {columns: _wave_time(m, n, columns, clusters) for columns in (256, 224, 192) if n % columns == 0}
        # narrower items cost about 2 % per flop: they are taken only where the waves promise 10 %
        if chosen != 256:
            assert candidates[chosen] < 0.90 * candidates[256]
        else:
            assert min(candidates.values()) >= 0.90 * candidates[256] - 1e-9
    if sm_count == 148:
        assert lib.fk_gemm_item_columns(8192, 3584, 8192, 0, 148) == 224   # 3.5 wave-times -> 3.06
        assert lib.fk_gemm_item_columns(8192, 28672, 8192, 0, 148) == 256
        assert lib.fk_gemm_item_columns(8192, 7168, 8192, 0, 148) == 256    # 6.5 -> 6.125: not enough
    # launches the narrow kernel takes keep the 256-column maps; so do shapes the tiling refuses
    assert lib.fk_gemm_item_columns(1024, 1792, 512, 0, 148) == 256
    assert lib.fk_gemm_item_columns(1024, 1792, 512, 16, 148) in (256, 224)
    assert lib.fk_gemm_item_columns(1000, 1792, 512, 0, 148) == 256


# ---------------------------------------------------------------- layouts

def test_packed_and_strided_strides():
    assert GlobalLayout.packed(BASE, [128, 256, 4]).strides == [2, 128 * 2, 256 * 128 * 2]
    assert GlobalLayout.strided(BASE, [128, 64], [1, 1024]).strides == [2, 1024 * 2]
    assert GlobalLayout.packed(BASE, [64, 8], FK_F32).strides == [4, 256]
    with pytest.raises(FerroKittensError, match="dimension 0 contiguously"):
        GlobalLayout.strided(BASE, [128, 64], [2, 256])
    with pytest.raises(FerroKittensError, match="rank 1 through 5"):
        GlobalLayout.packed(BASE, [2] * 6)


def test_the_box_is_one_subtile_and_higher_dimensions_select_it():
    layout = GlobalLayout.packed(BASE, [128, 256, 4])
    assert layout.descriptor_shape(64, 64) == ([128, 256, 4], [64, 64, 1])
    flat = GlobalLayout.packed(BASE, [64, 1024])
    assert flat.descriptor_shape(64, 128) == ([64, 1024], [64, 128])
    vector = GlobalLayout.packed(BASE, [128])
    assert vector.descriptor_shape(128, 1) == ([128], [128])
    with pytest.raises(FerroKittensError, match="rank-1 layout"):
        vector.descriptor_shape(64, 2)


def test_driver_requirements_name_the_field_that_violates_them():
    layout = GlobalLayout.packed(BASE, [64, 1024])
    extents, box = layout.descriptor_shape(64, 64)
    layout.check_driver_requirements(extents, box)
    narrow = GlobalLayout.packed(BASE, [4, 1024])
    narrow_extents, _ = narrow.descriptor_shape(64, 64)
    with pytest.raises(FerroKittensError, match=r"dimension 1.*multiple of 16"):
        narrow.check_driver_requirements(narrow_extents, box)
    with pytest.raises(FerroKittensError, match="16-byte aligned"):
        GlobalLayout.packed(BASE + 2, [64, 1024]).check_driver_requirements(extents, box)
    short = GlobalLayout.packed(BASE, [64, 16])
    short_extents, _ = short.descriptor_shape(64, 64)
    with pytest.raises(FerroKittensError, match="smaller than its box"):
        short.check_driver_requirements(short_extents, box)
    vector = GlobalLayout.packed(BASE, [64])
    vector_extents, legal = vector.descriptor_shape(8, 1)
    vector.check_driver_requirements(vector_extents, legal)
    with pytest.raises(FerroKittensError, match="box dimension 0 is 8 bytes"):
        vector.check_driver_requirements(vector_extents, [4])
    wide = GlobalLayout.packed(BASE, [1024, 1024])
    with pytest.raises(FerroKittensError, match="over the TMA maximum of 256"):
        wide.check_driver_requirements([1024, 1024], [512, 64])


def test_validation_happens_before_any_driver_call():
    """Bad arguments are refused on a machine with no GPU: nothing reaches the driver."""
    lib = library()
    with pytest.raises(FerroKittensError, match="16-byte aligned"):
        GlobalLayout.packed(BASE + 2, [64, 1024]).tensor_map(64)
    buffer = ctypes.create_string_buffer(256)
    aligned = (ctypes.addressof(buffer) + 63) & ~63
    assert lib.fk_encode_bf16_panels(aligned, BASE, 128, 128, 192, 2) == _lib.FK_ERR_SHAPE
    assert "whole number of 128-row boxes" in _lib.last_error()
    assert lib.fk_gemm_bf16_launch(aligned, aligned, aligned, 512, 256, 100, 8, None, None) == _lib.FK_ERR_SHAPE
    assert "does not divide the 256x256x64 tiling" in _lib.last_error()
    assert lib.fk_gemm_bf16_launch(aligned, aligned, aligned, 512, 256, 256, 0, None, None) == _lib.FK_ERR_SHAPE
    assert "group width of 0" in _lib.last_error()
    assert lib.fk_gemm_bf16_launch(None, aligned, aligned, 512, 256, 256, 8, None, None) == _lib.FK_ERR_INVALID
    assert lib.fk_flash_fwd_launch(aligned, aligned, aligned, aligned, None, None, 2, 192, 0.125, 1,
                                   None, None) == _lib.FK_ERR_SHAPE
    assert "does not divide the 128 queries" in _lib.last_error()
