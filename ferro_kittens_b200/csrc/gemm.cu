// bf16 GEMM  C[m, n] = sum_k A[m, k] * B[n, k]  (fp32 accumulate, bf16 out) for
// sm_100a: a persistent grid of two-CTA clusters, each pair sharing one
// tcgen05 M256 N256 K16 MMA (cta_group::2) that accumulates in tensor memory.
//
// Replaces the reference kernel `gemm_cg2_staged_x8x4` and its launcher
// (examples/src/gemm.rs:395-419, 477-538). Same operand layouts, same
// [256, 256] cluster tile, same `grouped` traversal; the structure is new:
//
//   warp 0      producer: this CTA's [128, 64] halves of A and B per k-block, by TMA,
//               into a kStages-deep SWIZZLE_128B ring; every load of the pair completes
//               on the leader CTA's `full` barrier (no multicast: the halves differ).
//   warp 1      (leader CTA only) MMA issue: 4 chained MMAs per k-block, tcgen05.commit
//               releases the stage in both CTAs, then hands the accumulator over.
//   warps 2-5   epilogue: tcgen05.ld -> bf16 -> SWIZZLE_128B staging -> TMA store,
//               one 32-row band per warp, double-buffered.
//
// Tensor memory holds two [128, 256] fp32 accumulators per CTA (all 512
// columns), so the epilogue of item i overlaps the main loop of item i+1.
// Barriers are initialised once per launch and their phases carried across
// items; roles meet only through them. Every wait is bounded.

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
namespace gemm {

constexpr uint32_t kBlockM = 128;   // rows of A (and of C) per CTA; the pair covers 256
constexpr uint32_t kBlockN = 256;   // columns of C per pair; each CTA stages kBlockN/2 rows of B
constexpr uint32_t kHalfN = kBlockN / 2;
constexpr uint32_t kBlockK = 64;    // one 128-byte swizzle atom of bf16
constexpr uint32_t kStages = 6;
constexpr uint32_t kAccumulators = 2;
constexpr uint32_t kTmemColumns = kAccumulators * kBlockN;  // 512
constexpr uint32_t kEpilogueWarps = 4;
constexpr uint32_t kStageColumns = 64;  // columns per epilogue pass: one swizzle atom of bf16
constexpr uint32_t kStageBuffers = 2;
constexpr uint32_t kThreads = (2 + kEpilogueWarps) * 32;
constexpr uint32_t kATileBytes = kBlockM * kBlockK * 2;
constexpr uint32_t kBTileBytes = kHalfN * kBlockK * 2;
constexpr uint32_t kBandBytes = 32 * kStageColumns * 2;  // one warp's [32, 64] bf16 staging tile
constexpr uint32_t kPairStageBytes = 2 * (kATileBytes + kBTileBytes);

// The shared plan, one walk for the kernel's offsets and the launch's total.
struct Plan {
    SharedPlan a_ring, b_ring, bands, full, empty, acc_full, acc_empty, tmem_slot, stop, end;
    constexpr Plan()
        : a_ring(SharedPlan{}.tile_ring(kBlockM, kBlockK, 2, kStages)),
          b_ring(a_ring.tile_ring(kHalfN, kBlockK, 2, kStages)),
          bands(b_ring.tile_ring(32, kStageColumns, 2, kEpilogueWarps * kStageBuffers)),
          full(bands.semaphores(kStages)),
          empty(full.semaphores(kStages)),
          acc_full(empty.semaphores(kAccumulators)),
          acc_empty(acc_full.semaphores(kAccumulators)),
          tmem_slot(acc_empty.tmem_slot()),
          stop(tmem_slot.word()),
          end(stop) {}
};
constexpr Plan kPlan{};
// Tiles must sit on 1024-byte boundaries for the operand descriptors' zero base
// offset; the kernel rounds its dynamic base up, which the launch pays for here.
constexpr uint32_t kBaseAlign = 1024;
constexpr uint32_t kSharedBytes = static_cast<uint32_t>(kPlan.end.bytes()) + kBaseAlign;
static_assert(kSharedBytes <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");
static_assert(kPlan.a_ring.at % 1024 == 0 && kPlan.b_ring.at % 1024 == 0 &&
                  kPlan.bands.at % 1024 == 0,
              "swizzled tiles must start on a 1024-byte boundary");

enum StallCode : uint32_t {
    kStallProducer = 0x101,
    kStallMmaFull = 0x102,
    kStallMmaAccumulator = 0x103,
    kStallEpilogue = 0x104,
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap a_map,
                          const __grid_constant__ CUtensorMap b_map,
                          const __grid_constant__ CUtensorMap c_map, uint32_t tiles_m,
                          uint32_t tiles_n, uint32_t group, uint32_t k_blocks, uint32_t* status) {
    extern __shared__ uint8_t dynamic_shared[];
    const uint32_t base = (smem_u32(dynamic_shared) + kBaseAlign - 1) & ~(kBaseAlign - 1);

    const uint32_t a_ring = base + kPlan.a_ring.at;
    const uint32_t b_ring = base + kPlan.b_ring.at;
    const uint32_t bands = base + kPlan.bands.at;
    const uint32_t full = base + kPlan.full.at;
    const uint32_t empty = base + kPlan.empty.at;
    const uint32_t acc_full = base + kPlan.acc_full.at;
    const uint32_t acc_empty = base + kPlan.acc_empty.at;
    const uint32_t slot = base + kPlan.tmem_slot.at;
    const uint32_t stop_addr = base + kPlan.stop.at;
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(
        dynamic_shared + (stop_addr - smem_u32(dynamic_shared)));
    volatile uint32_t* slot_ptr =
        reinterpret_cast<volatile uint32_t*>(dynamic_shared + (slot - smem_u32(dynamic_shared)));

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t peer = rank ^ 1u;
    const uint32_t items = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full + 8 * s, 1);
            mbar_init(empty + 8 * s, 1);
        }
        for (uint32_t a = 0; a < kAccumulators; ++a) {
            mbar_init(acc_full + 8 * a, 1);
            mbar_init(acc_empty + 8 * a, 2 * kEpilogueWarps);
        }
        *stop_flag = 0;
        fence_mbarrier_init();
        prefetch_tensormap(&a_map);
        prefetch_tensormap(&b_map);
        prefetch_tensormap(&c_map);
    }
    if (warp == 1) tmem_alloc<2>(slot, kTmemColumns);
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    tc_fence_after_sync();
    if (warp == 1) tmem_relinquish<2>();
    const uint32_t tmem = *slot_ptr;

    const StallSite site{status, stop_flag, mapa(stop_addr, peer)};

    if (warp == 0) {
        // ------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            uint32_t fill = 0;
            bool live = true;
            for (uint32_t item = cluster_id_x(); live && item < items; item += cluster_count_x()) {
                const TileCoord tile = grouped(item, tiles_m, tiles_n, group);
                const int a_row = static_cast<int>(2 * kBlockM * tile.row + kBlockM * rank);
                const int b_row = static_cast<int>(kBlockN * tile.column + kHalfN * rank);
                for (uint32_t k = 0; k < k_blocks; ++k, ++fill) {
                    const uint32_t s = fill % kStages;
                    const uint32_t parity = (fill / kStages) & 1u;
                    if (!mbar_wait(empty + 8 * s, parity ^ 1u, site, kStallProducer, fill)) {
                        live = false;
                        break;
                    }
                    // The leader's barrier collects all four boxes of the pair's stage.
                    const uint32_t arrive_at = mapa(full + 8 * s, 0);
                    if (rank == 0) mbar_arrive_expect_tx(full + 8 * s, kPairStageBytes);
                    const int column = static_cast<int>(kBlockK * k);
                    tma_load_2d_pair(a_ring + s * kATileBytes, &a_map, column, a_row, arrive_at);
                    tma_load_2d_pair(b_ring + s * kBTileBytes, &b_map, column, b_row, arrive_at);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue (leader only)
        if (rank == 0 && lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(2 * kBlockM, kBlockN, false, false);
            uint32_t drain = 0, count = 0;
            bool live = true;
            for (uint32_t item = cluster_id_x(); live && item < items;
                 item += cluster_count_x(), ++count) {
                const uint32_t acc = count % kAccumulators;
                const uint32_t acc_parity = (count / kAccumulators) & 1u;
                if (!mbar_wait(acc_empty + 8 * acc, acc_parity ^ 1u, site, kStallMmaAccumulator,
                               count)) {
                    live = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem + acc * kBlockN;
                for (uint32_t k = 0; k < k_blocks; ++k, ++drain) {
                    const uint32_t s = drain % kStages;
                    const uint32_t parity = (drain / kStages) & 1u;
                    if (!mbar_wait(full + 8 * s, parity, site, kStallMmaFull, drain)) {
                        live = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint64_t a_desc =
                        operand_descriptor(a_ring + s * kATileBytes, kKMajorLeadingBytes);
                    const uint64_t b_desc =
                        operand_descriptor(b_ring + s * kBTileBytes, kKMajorLeadingBytes);
#pragma unroll
                    for (uint32_t chunk = 0; chunk < kBlockK / 16; ++chunk) {
                        // Advancing the 14-bit address field by 32 B per K=16 chunk.
                        const uint64_t step = (chunk * kKMajorChunkBytes) >> 4;
                        mma_ss<2>(d_tmem, a_desc + step, b_desc + step, idesc, (k | chunk) != 0);
                    }
                    // The MMA's own retirement frees the stage, in both CTAs.
                    mma_commit<2>(empty + 8 * s);
                    mma_commit<2>(mapa(empty + 8 * s, 1));
                }
                if (!live) break;
                mma_commit<2>(acc_full + 8 * acc);
                mma_commit<2>(mapa(acc_full + 8 * acc, 1));
            }
        }
    } else {
        // ------------------------------------------------ epilogue (both CTAs)
        const uint32_t quadrant = warp & 3u;  // the tensor-memory lanes this warp may read
        const uint32_t my_bands = bands + (warp - 2) * kStageBuffers * kBandBytes;
        const uint32_t row_in_band = lane;
        uint32_t count = 0, pass = 0;
        bool live = true;
        for (uint32_t item = cluster_id_x(); live && item < items;
             item += cluster_count_x(), ++count) {
            const TileCoord tile = grouped(item, tiles_m, tiles_n, group);
            const uint32_t acc = count % kAccumulators;
            const uint32_t acc_parity = (count / kAccumulators) & 1u;
            if (!mbar_wait(acc_full + 8 * acc, acc_parity, site, kStallEpilogue, count)) {
                live = false;
                break;
            }
            tc_fence_after_sync();
            const int c_row =
                static_cast<int>(2 * kBlockM * tile.row + kBlockM * rank + 32 * quadrant);
            const int c_column = static_cast<int>(kBlockN * tile.column);
            const uint32_t t_row = tmem_address(tmem, 32 * quadrant, acc * kBlockN);
#pragma unroll 1
            for (uint32_t at = 0; at < kBlockN; at += kStageColumns, ++pass) {
                const uint32_t band = my_bands + (pass % kStageBuffers) * kBandBytes;
                // The store that last read this buffer must be done reading it.
                if (lane == 0) tma_store_wait_read<kStageBuffers - 1>();
                __syncwarp();
                uint32_t lo[32], hi[32];
                tmem_ld_32x32(t_row + at, lo);
                tmem_ld_32x32(t_row + at + 32, hi);
                tmem_wait_ld();
                if (at + kStageColumns == kBlockN) {
                    // Last read of this accumulator: hand it back to the MMA warp.
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(mapa(acc_empty + 8 * acc, 0));
                }
#pragma unroll
                for (uint32_t chunk = 0; chunk < 4; ++chunk) {
                    const uint32_t* v = lo + 8 * chunk;
                    st_shared_v4(band + swizzled_chunk_offset(row_in_band, chunk, 0),
                                 pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1])),
                                 pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3])),
                                 pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5])),
                                 pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7])));
                }
#pragma unroll
                for (uint32_t chunk = 0; chunk < 4; ++chunk) {
                    const uint32_t* v = hi + 8 * chunk;
                    st_shared_v4(band + swizzled_chunk_offset(row_in_band, 4 + chunk, 0),
                                 pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1])),
                                 pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3])),
                                 pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5])),
                                 pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7])));
                }
                // Every writer publishes to the async proxy, then one lane stores.
                fence_proxy_async_shared();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&c_map, band, c_column + static_cast<int>(at), c_row);
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    // ---------------------------------------------------- teardown
    if (*stop_flag) {
        // A role gave up: let copies and MMAs already in flight land before
        // shared and tensor memory are handed back.
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync();
    if (warp == 1) tmem_dealloc<2>(tmem, kTmemColumns);
}

}  // namespace gemm
}  // namespace fk

// ------------------------------------------------------------------ C ABI

using namespace fk;

extern "C" uint32_t fk_gemm_shared_bytes(void) { return gemm::kSharedBytes; }
extern "C" uint32_t fk_gemm_threads(void) { return gemm::kThreads; }

extern "C" uint32_t fk_gemm_grid(uint32_t m, uint32_t n, uint32_t sm_count) {
    const uint32_t tiles = (m / (2 * gemm::kBlockM)) * (n / gemm::kBlockN);
    const uint32_t clusters = sm_count / 2;
    return 2 * (tiles < clusters ? tiles : clusters);
}

extern "C" int fk_gemm_bf16_launch(const void* a_map, const void* b_map, const void* c_map,
                                   uint32_t m, uint32_t n, uint32_t k, uint32_t group, void* stream,
                                   uint32_t* device_status) {
    if (!a_map || !b_map || !c_map) return fk_fail(FK_ERR_INVALID, "a tensor map pointer is null");
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN ||
        k % gemm::kBlockK)
        return fk_fail(FK_ERR_SHAPE, "%ux%ux%u does not divide the %ux%ux%u tiling", m, n, k,
                       2 * gemm::kBlockM, gemm::kBlockN, gemm::kBlockK);
    if (group == 0)
        return fk_fail(FK_ERR_SHAPE, "a traversal group width of 0 has no tiles in it");

    int device = 0, sm_count = 0;
    FK_CUDA(cudaGetDevice(&device));
    FK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    uint32_t limit = 0;
    const int admitted = fk_admit_shared_plan(
        reinterpret_cast<const void*>(gemm::gemm_bf16_pair_kernel), gemm::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;

    const uint32_t grid = fk_gemm_grid(m, n, static_cast<uint32_t>(sm_count));
    gemm::gemm_bf16_pair_kernel<<<grid, gemm::kThreads, gemm::kSharedBytes,
                                  static_cast<cudaStream_t>(stream)>>>(
        *static_cast<const CUtensorMap*>(a_map), *static_cast<const CUtensorMap*>(b_map),
        *static_cast<const CUtensorMap*>(c_map), m / (2 * gemm::kBlockM), n / gemm::kBlockN, group,
        k / gemm::kBlockK, device_status);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

// The three maps `gemm::run` builds (examples/src/gemm.rs:506-513), plus the
// store map for C: dims [n, m] with the caller's leading dimension.
static int gemm_maps(const void* a, const void* b, void* c, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t ldc, CUtensorMap* maps) {
    fk_layout_t layout;
    const uint64_t a_extents[2] = {k, m}, b_extents[2] = {k, n}, c_extents[2] = {n, m};
    const uint64_t c_strides[2] = {1, ldc};
    int status = fk_layout_packed(&layout, reinterpret_cast<uint64_t>(a), FK_BF16, 2, a_extents);
    if (status == FK_OK) status = fk_tensor_map(&maps[0], &layout, gemm::kBlockK, gemm::kBlockM, FK_SWIZZLE_128B);
    if (status == FK_OK) status = fk_layout_packed(&layout, reinterpret_cast<uint64_t>(b), FK_BF16, 2, b_extents);
    if (status == FK_OK) status = fk_tensor_map(&maps[1], &layout, gemm::kBlockK, gemm::kHalfN, FK_SWIZZLE_128B);
    if (status == FK_OK) status = fk_layout_strided(&layout, reinterpret_cast<uint64_t>(c), FK_BF16, 2, c_extents, c_strides);
    if (status == FK_OK) status = fk_tensor_map(&maps[2], &layout, gemm::kStageColumns, 32, FK_SWIZZLE_128B);
    return status;
}

extern "C" int fk_gemm_bf16(const void* a, const void* b, void* c, uint32_t m, uint32_t n,
                            uint32_t k, uint32_t ldc, uint32_t group, void* stream,
                            uint32_t* device_status) {
    if (!a || !b || !c) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN ||
        k % gemm::kBlockK)
        return fk_fail(FK_ERR_SHAPE, "%ux%ux%u does not divide the %ux%ux%u tiling", m, n, k,
                       2 * gemm::kBlockM, gemm::kBlockN, gemm::kBlockK);
    if (ldc < n) return fk_fail(FK_ERR_SHAPE, "ldc %u is narrower than the %u columns of C", ldc, n);
    alignas(64) CUtensorMap maps[3];
    const int status = gemm_maps(a, b, c, m, n, k, ldc, maps);
    if (status != FK_OK) return status;
    return fk_gemm_bf16_launch(&maps[0], &maps[1], &maps[2], m, n, k, group, stream, device_status);
}

extern "C" int fk_gemm_bf16_host(const uint16_t* a_host, const uint16_t* b_host, uint16_t* c_host,
                                 uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    if (!a_host || !b_host || !c_host) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    const size_t a_bytes = size_t(m) * k * 2, b_bytes = size_t(n) * k * 2, c_bytes = size_t(m) * n * 2;
    void *a = nullptr, *b = nullptr, *c = nullptr;
    uint32_t* status_words = nullptr;
    int status = scratch(0, a_bytes, &a);
    if (status == FK_OK) status = scratch(1, b_bytes, &b);
    if (status == FK_OK) status = scratch(2, c_bytes, &c);
    if (status == FK_OK) status = scratch_status(&status_words);
    if (status != FK_OK) return status;
    cudaStream_t stream = nullptr;
    FK_CUDA(cudaMemsetAsync(status_words, 0, 16, stream));
    FK_CUDA(cudaMemcpyAsync(a, a_host, a_bytes, cudaMemcpyHostToDevice, stream));
    FK_CUDA(cudaMemcpyAsync(b, b_host, b_bytes, cudaMemcpyHostToDevice, stream));
    status = fk_gemm_bf16(a, b, c, m, n, k, n, group, stream, status_words);
    if (status != FK_OK) return status;
    FK_CUDA(cudaMemcpyAsync(c_host, c, c_bytes, cudaMemcpyDeviceToHost, stream));
    return fk_status_check(status_words, stream);
}
