// Host+device address arithmetic shared by the kernels, the launchers and
// the CPU unit tests: the tile traversal, SWIZZLE_128B chunk addresses, the
// tcgen05 shared-memory operand descriptor and instruction descriptor, and the
// shared-memory plan cursor. Everything is constexpr, so the byte total a launch
// declares and the offsets a kernel uses come from the same walk.
#pragma once

#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define FK_HD __host__ __device__ __forceinline__
#else
#define FK_HD inline
#endif

namespace fk {

// ---------------------------------------------------------------- traversal

struct TileCoord {
    uint32_t row, column;
};

/// Work item -> (tile row, tile column) of a rows x columns grid, walking
/// `group` tile-rows at a time; the last group is short when `group` does not
/// divide `rows`. Same map as the reference's `pipeline::grouped`
/// (src/pipeline.rs:207-213): group 1 is row-major, group >= rows column-major.
FK_HD constexpr TileCoord grouped(uint32_t item, uint32_t rows, uint32_t columns, uint32_t group) {
    const uint32_t span = group * columns;
    const uint32_t first = item / span * group;
    const uint32_t left = rows - first;
    const uint32_t height = group < left ? group : left;
    const uint32_t within = item % span;
    return TileCoord{first + within % height, within / height};
}

// ---------------------------------------------------------------- swizzle

/// Byte offset, from a tile base whose 128-byte-row phase is `phase`, of
/// 16-byte chunk `chunk` (0..7) of 128-byte row `row` under SWIZZLE_128B
/// (reference: `SwizzledChunks::at`, src/shared.rs:1341-1348).
FK_HD constexpr uint32_t swizzled_chunk_offset(uint32_t row, uint32_t chunk, uint32_t phase) {
    return row * 128u + ((chunk ^ ((row + phase) & 7u)) << 4);
}

// ---------------------------------------------------------------- descriptors

/// tcgen05 shared-memory operand descriptor for a SWIZZLE_128B tile:
/// address>>4 in [13:0], leading byte offset>>4 in [29:16], stride byte offset
/// 1024>>4 in [45:32], the fixed 0b001 at [48:46], swizzle mode 2 at [63:61]
/// (reference: `encode_descriptor`, src/shared.rs:1251-1258).
FK_HD constexpr uint64_t operand_descriptor(uint64_t shared_address, uint32_t leading_bytes) {
    return ((shared_address >> 4) & 0x3fffull) | ((uint64_t)((leading_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((1024u >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}
/// Leading byte offset of a K-major operand (ignored by the hardware under a swizzle).
constexpr uint32_t kKMajorLeadingBytes = 16;
/// Bytes between consecutive K=16 chunks inside one 64-element swizzle atom row.
constexpr uint32_t kKMajorChunkBytes = 32;
/// Bytes between consecutive K=16 chunks of an MN-major operand: 16 rows of 128 B.
constexpr uint32_t kMnMajorChunkBytes = 2048;

/// tcgen05 instruction descriptor, kind::f16 with bf16 operands and an fp32
/// accumulator: D format at [5:4], A/B formats at [9:7]/[12:10], transpose
/// A/B at 15/16, N>>3 at [22:17], M>>4 at [28:24]
/// (reference: `descriptor` src/mma.rs:137-146, layout restated in its test :576-584).
/// `operand_format`: 1 = bf16 (the default), 0 = fp16, for both A and B.
FK_HD constexpr uint32_t instruction_descriptor(uint32_t m, uint32_t n, bool transpose_a,
                                                bool transpose_b, uint32_t operand_format = 1u) {
    return (1u << 4) | (operand_format << 7) | (operand_format << 10) |
           ((transpose_a ? 1u : 0u) << 15) | ((transpose_b ? 1u : 0u) << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}

/// Tensor-memory address of (lane row, 32-bit column) from an allocation base
/// (reference: `TmemTile::at`, src/tmem.rs:487).
FK_HD constexpr uint32_t tmem_address(uint32_t base, uint32_t row, uint32_t column) {
    return base + (row << 16) + column;
}

// ---------------------------------------------------------------- shared plan

/// Cursor over a launch's dynamic shared memory. Each reservation is aligned
/// to its own type's rule (tiles 128, barriers 8, tensor-memory slot 4) and the
/// running total is what the launch declares. Mirrors the reference's
/// `SharedPlan` (src/plan.rs:73-304) with the tile shapes as value parameters.
struct SharedPlan {
    static constexpr size_t kTileAlign = 128;
    static constexpr size_t kBarrierBytes = 8;
    static constexpr size_t kBarrierAlign = 8;
    static constexpr size_t kTmemSlotBytes = 4;

    size_t offset = 0;
    size_t at = 0;  // start of the last reservation

    FK_HD constexpr size_t bytes() const { return offset; }

    FK_HD constexpr SharedPlan reserve(size_t size, size_t align) const {
        const size_t start = (offset + align - 1) / align * align;
        return SharedPlan{start + size, start};
    }
    FK_HD constexpr SharedPlan tile(size_t rows, size_t columns, size_t element_bytes) const {
        return reserve(rows * columns * element_bytes, kTileAlign);
    }
    FK_HD constexpr SharedPlan tile_ring(size_t rows, size_t columns, size_t element_bytes,
                                         size_t count) const {
        return reserve(rows * columns * element_bytes * count, kTileAlign);
    }
    FK_HD constexpr SharedPlan semaphores(size_t count) const {
        return reserve(count * kBarrierBytes, kBarrierAlign);
    }
    FK_HD constexpr SharedPlan semaphore() const { return semaphores(1); }
    FK_HD constexpr SharedPlan tmem_slot() const { return reserve(kTmemSlotBytes, 4); }
    FK_HD constexpr SharedPlan word() const { return reserve(4, 4); }
};

}  // namespace fk
