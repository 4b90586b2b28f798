// ferro_kittens.hpp -- the crate's host surface, spelled in C++ over the C ABI.
//
// ferro-kittens' callers are compiled code (Rust); where that toolchain is not
// available this header is the host side a caller writes against: the same
// names, argument meaning and error behaviour as the crate's `global`, `plan`,
// `launch`, `watchdog` modules and its two kernel launchers, each a thin inline
// wrapper over `ferro_kittens.h`. Header-only, C++17, no CUDA headers needed.
#pragma once

#include <array>
#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <type_traits>

#include "ferro_kittens.h"

namespace kittens {

/// What `Result<_, Box<dyn Error>>` carries in the crate: the message names the violated field.
struct Error : std::runtime_error {
    int code;
    Error(int code_, const std::string& what) : std::runtime_error(what), code(code_) {}
};

inline void check(int code) {
    if (code != FK_OK) throw Error(code, fk_last_error());
}

// ---------------------------------------------------------------- shared (the tile types a map is built for)
namespace shared {

struct Bf16 { static constexpr uint32_t ELEMENT = FK_BF16; static constexpr std::size_t BYTES = 2; };
struct F16 { static constexpr uint32_t ELEMENT = FK_F16; static constexpr std::size_t BYTES = 2; };
struct F32 { static constexpr uint32_t ELEMENT = FK_F32; static constexpr std::size_t BYTES = 4; };
struct Swizzle128B { static constexpr std::size_t ATOM_BYTES = 128; };

/// `SharedTile<E, R, C, Swizzle128B>` (src/shared.rs:544-615) as far as the host needs it: the
/// box one TMA instruction delivers is one [R, 128 bytes] subtile (src/global.rs:1717-1725).
template <class E, std::size_t R, std::size_t C, class S = Swizzle128B>
struct SharedTile {
    using Element = E;
    static constexpr std::size_t SUBTILE_COLS = S::ATOM_BYTES / E::BYTES;
    static constexpr std::size_t SUBTILES = C / SUBTILE_COLS;
    static constexpr std::size_t SUBTILE_BYTES = R * S::ATOM_BYTES;
    static constexpr std::size_t BYTES = R * C * E::BYTES;
    static constexpr std::size_t BOX_COLS = SUBTILE_COLS;
    static constexpr std::size_t BOX_ROWS = R;
    static constexpr uint32_t SWIZZLE = FK_SWIZZLE_128B;
};

}  // namespace shared

// ---------------------------------------------------------------- global (src/global.rs:1649-2076)
namespace global {

/// The 128 opaque bytes a kernel's tensor-map parameter is copied from (`TensorMap`, :2022-2031).
/// Lives on the host: the kernels take the map by value, so there is nothing to upload.
struct alignas(64) TensorMap {
    unsigned char opaque[128];
    const void* as_ptr() const { return opaque; }
};
using PanelMap = TensorMap;

/// `GlobalLayout<E, RANK>`: a RANK-dimensional buffer, dimension 0 contiguous (a row-major
/// [rows, columns] matrix is extents {columns, rows}). Does not own or borrow the buffer.
template <class E, std::size_t RANK>
class GlobalLayout {
    static_assert(RANK >= 1 && RANK <= 5, "cuTensorMapEncodeTiled describes rank 1 through 5");
    fk_layout_t raw_{};

   public:
    static GlobalLayout packed(uint64_t base, const std::array<uint64_t, RANK>& extents) {
        GlobalLayout layout;
        check(fk_layout_packed(&layout.raw_, base, E::ELEMENT, RANK, extents.data()));
        return layout;
    }
    static GlobalLayout strided(uint64_t base, const std::array<uint64_t, RANK>& extents,
                                const std::array<uint64_t, RANK>& element_strides) {
        GlobalLayout layout;
        check(fk_layout_strided(&layout.raw_, base, E::ELEMENT, RANK, extents.data(), element_strides.data()));
        return layout;
    }
    std::array<uint64_t, RANK> strides() const {
        std::array<uint64_t, RANK> out{};
        for (std::size_t d = 0; d < RANK; ++d) out[d] = raw_.strides_bytes[d];
        return out;
    }
    /// `descriptor_shape::<T>` (:1867-1888): globalDim and boxDim for a map delivering `Tile`.
    template <class Tile>
    void descriptor_shape(std::array<uint64_t, RANK>& extents, std::array<uint32_t, RANK>& box) const {
        uint64_t e[5];
        uint32_t b[5];
        check(fk_layout_descriptor_shape(&raw_, Tile::BOX_COLS, Tile::BOX_ROWS, e, b));
        for (std::size_t d = 0; d < RANK; ++d) { extents[d] = e[d]; box[d] = b[d]; }
    }
    /// `tensor_map::<T>` (:1920-1964): every field but the buffer comes from the tile type.
    template <class Tile>
    TensorMap tensor_map() const {
        static_assert(std::is_same<typename Tile::Element, E>::value, "the tile and the layout disagree on the element");
        TensorMap map;
        check(fk_tensor_map(map.opaque, &raw_, Tile::BOX_COLS, Tile::BOX_ROWS, Tile::SWIZZLE));
        return map;
    }
};

/// `encode_bf16_panels::<R, C>` (:2067-2076): rank-3 map over packed [planes, rows, C] bf16.
template <std::size_t R, std::size_t C>
inline PanelMap encode_bf16_panels(uint64_t base, uint64_t rows, uint64_t planes) {
    PanelMap map;
    check(fk_encode_bf16_panels(map.opaque, base, R, C, rows, planes));
    return map;
}

}  // namespace global

// ---------------------------------------------------------------- plan (src/plan.rs:73-304)
namespace plan {

/// The cursor over a launch's dynamic shared memory; every reservation aligns to its own rule.
class SharedPlan {
    std::size_t offset_ = 0;

   public:
    static constexpr std::size_t TILE_ALIGN = 128, BARRIER_BYTES = 8, BARRIER_ALIGN = 8, TMEM_SLOT_BYTES = 4;
    static constexpr SharedPlan sizing() { return SharedPlan{}; }
    constexpr std::size_t bytes() const { return offset_; }
    /// Returns the start of the run and advances the cursor.
    constexpr std::size_t reserve(std::size_t size, std::size_t align) {
        const std::size_t at = (offset_ + align - 1) / align * align;
        offset_ = at + size;
        return at;
    }
    template <class Tile>
    constexpr std::size_t tile() { return reserve(Tile::BYTES, TILE_ALIGN); }
    template <class Tile, std::size_t N>
    constexpr std::size_t tile_ring() { return reserve(Tile::BYTES * N, TILE_ALIGN); }
    constexpr std::size_t semaphores(std::size_t count) { return reserve(count * BARRIER_BYTES, BARRIER_ALIGN); }
    constexpr std::size_t semaphore() { return semaphores(1); }
    constexpr std::size_t tmem_slot() { return reserve(TMEM_SLOT_BYTES, 4); }
};

}  // namespace plan

// ---------------------------------------------------------------- launch (src/launch.rs:23-132)
namespace launch {

struct SharedPlanTooLarge : Error {
    uint32_t bytes, limit;
    SharedPlanTooLarge(uint32_t bytes_, uint32_t limit_)
        : Error(FK_ERR_TOO_LARGE, fk_last_error()), bytes(bytes_), limit(limit_) {}
};

/// Opt `kernel` into `bytes` of dynamic shared memory; idempotent, never lowers.
inline void admit_shared_plan(const void* kernel, uint32_t bytes) {
    uint32_t limit = 0;
    const int code = fk_admit_shared_plan(kernel, bytes, &limit);
    if (code == FK_ERR_TOO_LARGE) throw SharedPlanTooLarge(bytes, limit);
    check(code);
}

}  // namespace launch

// ---------------------------------------------------------------- watchdog (src/watchdog.rs:300-332)
namespace watchdog {

constexpr uint32_t DEFAULT_BUDGET_MS = 30000;
/// Returns an error (FK_ERR_TIMEOUT) where the crate aborts the process.
inline void wait(void* stream, uint32_t budget_ms = DEFAULT_BUDGET_MS) { check(fk_wait_stream(stream, budget_ms)); }
inline void wait_event(void* event, uint32_t budget_ms = DEFAULT_BUDGET_MS) { check(fk_wait_event(event, budget_ms)); }

}  // namespace watchdog

// ---------------------------------------------------------------- the two launchers
namespace gemm {

constexpr std::size_t BLOCK_M = 128, BLOCK_N = 256, HALF_N = 128, BLOCK_K = 64;
constexpr uint32_t GROUP = FK_GEMM_GROUP;  // the reference ships 8 for its kernel (examples/src/gemm.rs:138)
using ATile = shared::SharedTile<shared::Bf16, BLOCK_M, BLOCK_K>;
using BTile = shared::SharedTile<shared::Bf16, HALF_N, BLOCK_K>;
using CStage = shared::SharedTile<shared::Bf16, 32, 64>;

inline uint32_t grid(uint32_t m, uint32_t n, uint32_t sm_count = 148) { return fk_gemm_grid(m, n, sm_count); }

/// `gemm::run` between staging and read-back (examples/src/gemm.rs:506-536): build the maps,
/// launch on `stream`. `status` is null or 4 zeroed device words (see fk_status_check).
/// `flags`: FK_GEMM_F16_OPERANDS for fp16 A and B (examples/src/gemm_sol.rs), FK_GEMM_ACCUMULATE
/// for C += A.B^T through the copy engine's reduce-add (src/shared.rs:974-1009), FK_GEMM_RELU for
/// max(x, 0) before the rounding (src/reg.rs:261). `bias`: 0 or the device address of n bf16 values
/// added per column in fp32 before the rounding (src/global.rs:410-416).
inline void run(void* stream, uint64_t a, uint64_t b, uint64_t c, uint32_t m, uint32_t n, uint32_t k,
                uint32_t group = GROUP, uint32_t* status = nullptr, uint32_t flags = 0, uint64_t bias = 0) {
    global::TensorMap a_map, b_map;
    if (flags & FK_GEMM_F16_OPERANDS) {
        using A16 = shared::SharedTile<shared::F16, BLOCK_M, BLOCK_K>;
        using B16 = shared::SharedTile<shared::F16, HALF_N, BLOCK_K>;
        a_map = global::GlobalLayout<shared::F16, 2>::packed(a, {k, m}).tensor_map<A16>();
        b_map = global::GlobalLayout<shared::F16, 2>::packed(b, {k, n}).tensor_map<B16>();
    } else {
        a_map = global::GlobalLayout<shared::Bf16, 2>::packed(a, {k, m}).tensor_map<ATile>();
        b_map = global::GlobalLayout<shared::Bf16, 2>::packed(b, {k, n}).tensor_map<BTile>();
    }
    const auto c_map = global::GlobalLayout<shared::Bf16, 2>::packed(c, {n, m}).tensor_map<CStage>();
    check(fk_gemm_launch_fused(a_map.as_ptr(), b_map.as_ptr(), c_map.as_ptr(), reinterpret_cast<const void*>(bias),
                               m, n, k, group, flags, stream, status));
}

}  // namespace gemm

namespace flash_forward {

constexpr std::size_t QUERIES = 128, KEYS = 128, HEAD = 128;
constexpr float SCALE = 0.125f;  // examples/src/flash_forward.rs:321

/// `flash_forward::run` between staging and read-back (examples/src/flash_forward.rs:498-529),
/// with the widened signature: planes, causal flag, bf16 or fp32 output, optional LSE.
inline void run(void* stream, uint64_t q, uint64_t k, uint64_t v, uint64_t o_bf16, float* o_f32, float* lse,
                uint32_t planes, uint32_t sequence, float scale, bool causal, uint32_t* status = nullptr) {
    const auto q_map = global::encode_bf16_panels<QUERIES, HEAD>(q, sequence, planes);
    const auto k_map = global::encode_bf16_panels<KEYS, HEAD>(k, sequence, planes);
    const auto v_map = global::encode_bf16_panels<KEYS, HEAD>(v, sequence, planes);
    check(fk_flash_fwd_launch(q_map.as_ptr(), k_map.as_ptr(), v_map.as_ptr(), reinterpret_cast<void*>(o_bf16),
                              o_bf16 ? nullptr : o_f32, lse, planes, sequence, scale, causal ? 1 : 0, stream, status));
}

}  // namespace flash_forward

/// Flash-attention backward (no kernel of this name in the crate; see fk_flash_bwd): gradients of
/// `flash_forward::run` with respect to q, k, v from its output and log-sum-exp. `workspace` holds
/// `workspace_floats(planes, sequence)` floats on the device.
namespace flash_backward {

inline std::size_t workspace_floats(uint32_t planes, uint32_t sequence) {
    return static_cast<std::size_t>(fk_flash_bwd_workspace_bytes(planes, sequence) / sizeof(float));
}
inline void run(void* stream, uint64_t q, uint64_t k, uint64_t v, uint64_t o, uint64_t d_o, const float* lse,
                uint64_t dq, uint64_t dk, uint64_t dv, float* workspace, uint32_t planes, uint32_t sequence,
                float scale, bool causal, uint32_t* status = nullptr) {
    check(fk_flash_bwd(reinterpret_cast<const void*>(q), reinterpret_cast<const void*>(k),
                       reinterpret_cast<const void*>(v), reinterpret_cast<const void*>(o),
                       reinterpret_cast<const void*>(d_o), lse, reinterpret_cast<void*>(dq),
                       reinterpret_cast<void*>(dk), reinterpret_cast<void*>(dv), workspace, planes, sequence, scale,
                       causal ? 1 : 0, stream, status));
}

}  // namespace flash_backward

/// The row kernels (examples/src/softmax.rs, examples/src/layernorm.rs), over rows of 128 bf16 columns.
namespace rows {

constexpr std::size_t ROWS = 128, COLUMNS = 128;
constexpr float EPSILON = 1e-5f;  // examples/src/layernorm.rs:313

inline void softmax_rows(void* stream, uint64_t source, uint64_t destination, uint32_t rows_per_plane,
                         uint32_t planes, uint32_t* status = nullptr) {
    check(fk_softmax_rows(reinterpret_cast<const void*>(source), reinterpret_cast<void*>(destination), rows_per_plane,
                          planes, stream, status));
}
inline void layernorm_rows(void* stream, uint64_t source, uint64_t gamma, uint64_t beta, uint64_t destination,
                           uint32_t row_count, float epsilon = EPSILON, uint32_t* status = nullptr) {
    check(fk_layernorm_rows(reinterpret_cast<const void*>(source), reinterpret_cast<const void*>(gamma),
                            reinterpret_cast<const void*>(beta), reinterpret_cast<void*>(destination), row_count,
                            epsilon, stream, status));
}
inline void groupnorm_tile(void* stream, uint64_t source, uint64_t destination, uint32_t row_count,
                           float epsilon = EPSILON, uint32_t* status = nullptr) {
    check(fk_groupnorm_tile(reinterpret_cast<const void*>(source), reinterpret_cast<void*>(destination), row_count,
                            epsilon, stream, status));
}

}  // namespace rows

}  // namespace kittens
