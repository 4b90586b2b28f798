// bf16 GEMM  C[m, n] = sum_k A[m, k] * B[n, k]  (fp32 accumulate, bf16 out) for
// sm_100a: a persistent grid of two-CTA clusters, each pair sharing tcgen05
// M256 N256 K16 MMAs (cta_group::2) that accumulate in tensor memory.
//
// Replaces the reference kernel `gemm_cg2_staged_x8x4` and its launcher
// (examples/src/gemm.rs:395-419, 477-538). Same operand layouts and the same
// `grouped` traversal; the structure is new:
//
//   item        one [512, 256] block of C per cluster: two vertically adjacent [256, 256] pair
//               tiles ("halves") that share every B tile, each half accumulating in its own
//               256 tensor-memory columns. Per k-block a CTA stages two [128, 64] tiles of A
//               and one [128, 64] tile of B: 48 KiB for 1024 tensor cycles, against 32 KiB for
//               512 with a single [256, 256] tile -- what keeps the operand feed under the
//               L2->SM rate without multicast. The last partial wave of a launch is re-cut
//               into single-half items when that shortens it, and a launch whose tile count sits
//               just past a whole number of waves takes narrower items ([512, 224] or [512, 192],
//               the MMA's N) when those fill the waves better.
//   warp 0      producer: this CTA's A and B tiles per k-block, by TMA, into a kStages-deep
//               SWIZZLE_128B ring; every load of the pair completes on the leader's `full`.
//   warp 1      (leader CTA only) MMA issue: 4 chained MMAs per half per k-block;
//               tcgen05.commit releases the stage in both CTAs, then publishes the accumulators.
//   warps 2-9   epilogue: warps 2-5 drain half 0, warps 6-9 half 1, one 32-row band each:
//               tcgen05.ld -> bf16 pairs held in registers -> accumulator handed back ->
//               SWIZZLE_128B staging -> TMA store, overlapping the next item's main loop.
//
//   warp 10     (leader CTA only, launches of more items than resident clusters) the item feed: the
//               grid has one cluster per item, the resident clusters never exit, and this warp asks
//               the hardware for the next cluster that has not started (cluster launch control),
//               one item ahead, and publishes its index to every role of both CTAs. The items in
//               flight are therefore always the next ones of the traversal, however far the
//               clusters' speeds drift apart over a launch: a static round-robin lets slow clusters
//               fall waves behind, and the operand panels live in L2 multiply. (The reference's
//               stealing item loop, `run_stealing` over a `ClcQueue`, src/pipeline.rs:276-660, which
//               its `gemm_sol` runs on, examples/src/gemm_sol.rs:289-321; it asks after an item,
//               with the answer multicast to the cluster; here the request goes out an item ahead
//               and the leader forwards the answer, so no role ever waits for it.)
//
// Barriers are initialised once per launch and their phases carried across
// items; roles meet only through them. Every wait is bounded.
//
// Launches under one wave (fewer items than clusters) can split K across the idle
// clusters (the `true` instantiation): every unit accumulates a run of k-blocks of one
// item, adds its fp32 tile into a caller-owned workspace through the copy engine's
// reduce-add, and the unit that arrives last on the band's counter reads the sums back,
// applies bias / ReLU, rounds ONCE to bf16 and stores -- and leaves the workspace zero.

#include <mutex>

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
namespace gemm {

constexpr uint32_t kBlockM = 128;   // rows of A (and of C) per CTA per half; the pair covers 256
constexpr uint32_t kHalves = 2;     // [256, 256] pair tiles per item, stacked along M
constexpr uint32_t kBlockN = 256;   // columns of C per item; each CTA stages kBlockN/2 rows of B
constexpr uint32_t kHalfN = kBlockN / 2;
constexpr uint32_t kBlockK = 64;    // one 128-byte swizzle atom of bf16
constexpr uint32_t kStages = 4;
constexpr uint32_t kTmemColumns = kHalves * kBlockN;  // 512
constexpr uint32_t kEpilogueWarps = 4 * kHalves;
constexpr uint32_t kStageColumns = 64;  // columns per epilogue pass: one swizzle atom of bf16
constexpr uint32_t kPasses = kBlockN / kStageColumns;
// What an item's fourth epilogue pass is: 64 columns (items 256 wide), 32 (224) or nothing (192).
enum LastPass : uint32_t { kLastNone = 0, kLastNarrow = 1, kLastWhole = 2 };
constexpr uint32_t kFeedWarp = 2 + kEpilogueWarps;
constexpr uint32_t kThreads = (3 + kEpilogueWarps) * 32;
// The item feed: a ring of item indices every role reads in turn. Its readers are, per CTA, the
// producer thread and the epilogue warps, and the leader's MMA thread.
constexpr uint32_t kFeedSlots = 2;
constexpr uint32_t kFeedReaders = 2 * (1 + kEpilogueWarps) + 1;
constexpr uint32_t kNoItem = 0xffffffffu;
constexpr uint32_t kATileBytes = kBlockM * kBlockK * 2;
constexpr uint32_t kBTileBytes = kHalfN * kBlockK * 2;
constexpr uint32_t kBandBytes = 32 * kStageColumns * 2;  // one warp's [32, 64] bf16 staging tile

// The shared plan, one walk for the kernel's offsets and the launch's total.
struct Plan {
    SharedPlan a_ring, b_ring, bands, full, empty, acc_full, acc_empty, feed_full, feed_empty, feed_go, claim_full,
        claim_answer, feed_ring, tmem_slot, stop, end;
    constexpr Plan()
        : a_ring(SharedPlan{}.tile_ring(kBlockM, kBlockK, 2, kStages * kHalves)),
          b_ring(a_ring.tile_ring(kHalfN, kBlockK, 2, kStages)),
          bands(b_ring.tile_ring(32, kStageColumns, 2, kEpilogueWarps)),
          full(bands.semaphores(kStages)),
          empty(full.semaphores(kStages)),
          acc_full(empty.semaphore()),
          acc_empty(acc_full.semaphore()),
          feed_full(acc_empty.semaphores(kFeedSlots)),
          feed_empty(feed_full.semaphores(kFeedSlots)),
          feed_go(feed_empty.semaphore()),
          claim_full(feed_go.semaphore()),
          claim_answer(claim_full.reserve(16, 16)),
          feed_ring(claim_answer.reserve(4 * kFeedSlots, 4)),
          tmem_slot(feed_ring.tmem_slot()),
          stop(tmem_slot.word()),
          end(stop) {}
};
constexpr Plan kPlan{};
// Tiles must sit on 1024-byte boundaries for the operand descriptors' zero base
// offset: the dynamic shared array is declared with that alignment and the kernel
// refuses to run (status kMisaligned) should the base ever come back otherwise.
constexpr uint32_t kBaseAlign = 1024;
constexpr uint32_t kSharedBytes = static_cast<uint32_t>(kPlan.end.bytes());
static_assert(kSharedBytes <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");
static_assert(kEpilogueWarps * kPasses * kBandBytes <= kStages * kHalves * kATileBytes,
              "the last item stages every pass of every epilogue warp in the A ring");
static_assert(kPlan.a_ring.at % 1024 == 0 && kPlan.b_ring.at % 1024 == 0 &&
                  kPlan.bands.at % 1024 == 0,
              "swizzled tiles must start on a 1024-byte boundary");

enum StallCode : uint32_t {
    kStallProducer = 0x101,
    kStallMmaFull = 0x102,
    kStallMmaAccumulator = 0x103,
    kStallEpilogue = 0x104,
    kStallFeed = 0x105,
    kStallClaim = 0x106,
    kMisaligned = 0x1ff,
};

// What the launch hands every role so that each walks the same item list.
struct Schedule {
    uint32_t m;          // rows of C
    uint32_t tiles_m;    // [512, 256] tile rows: ceil(m / 512)
    uint32_t tiles_n;    // tile columns: n / tile_n
    uint32_t tile_n;     // columns of C per item (the MMAs' N): 256, or 224 / 192 where that fills the waves better
    uint32_t group;      // traversal width of `grouped`
    uint32_t k_blocks;   // k / 64
    uint32_t dynamic;    // non-zero: one cluster per item in the grid, items handed out by the feed warp
    uint32_t whole;      // leading items that are whole two-half tiles
    uint32_t items;      // whole + 2 * (tiles - whole): the rest are single halves
    uint32_t idesc;      // tcgen05 instruction descriptor (operand format differs by entry point)
    uint32_t accumulate; // non-zero: C += A . B^T through the copy engine's reduce-add
    uint32_t relu;       // non-zero: max(x, 0) on the fp32 value before it is rounded
    const uint16_t* bias;  // null, or n bf16 values added per column in fp32 before rounding
    // K split across clusters (launches under one wave; the kernel's `true` instantiation):
    uint32_t splits;       // units per item; 1 everywhere else
    uint32_t split_blocks; // k-blocks per unit
    uint32_t n;            // columns of C: the row pitch of `partial`
    float* partial;        // fp32 [m, n] sums, zero before and after a launch
    uint32_t* arrivals;    // units that have added their tile, per (item, CTA rank, epilogue warp); zero likewise
};

struct Item {
    uint32_t row;     // first row of C the item covers
    uint32_t column;  // first column
    uint32_t halves;  // 0 (nothing inside the matrix), 1 or 2
};

__host__ __device__ __forceinline__ Item item_at(const Schedule& plan, uint32_t index) {
    uint32_t tile = index, first_half = 0, halves = kHalves;
    if (index >= plan.whole) {
        const uint32_t rest = index - plan.whole;
        tile = plan.whole + rest / kHalves;
        first_half = rest % kHalves;
        halves = 1;
    }
    const TileCoord at = grouped(tile, plan.tiles_m, plan.tiles_n, plan.group);
    Item item;
    item.row = kHalves * 2 * kBlockM * at.row + 2 * kBlockM * first_half;
    item.column = plan.tile_n * at.column;
    item.halves = item.row >= plan.m ? 0u
                  : (halves == 2 && item.row + 2 * kBlockM >= plan.m) ? 1u
                                                                       : halves;
    return item;
}

// The fused epilogue on one pass of a band (a column-vector bias and a unary map on the register
// tile, src/global.rs:410-416, src/reg.rs:261), then the ONE rounding to bf16: `lo` and `hi` hold
// this lane's row, columns [column, column + 32) and [column + 32, column + 64) as fp32 bits;
// every lane holds the same columns, so the bias words are broadcast loads. `parts` == 1 is the
// 32-column pass that ends an item whose width is not a multiple of 64: only `lo` is real then
// (the bias is not read past it) and only the first 16 words of `packed` mean anything.
__device__ __forceinline__ void finish_pass(uint32_t (&lo)[32], uint32_t (&hi)[32], const Schedule& plan,
                                            uint32_t column, uint32_t (&packed)[32], uint32_t parts = 2) {
    if (plan.bias || plan.relu) {
        const float floor = plan.relu ? 0.0f : -INFINITY;
#pragma unroll
        for (uint32_t part = 0; part < 2; ++part) {
            if (part >= parts) break;
            uint32_t* const values = part ? hi : lo;
            uint32_t words[16];
            if (plan.bias) {
                const uint4* source = reinterpret_cast<const uint4*>(plan.bias + column + 32 * part);
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q) {
                    const uint4 v = __ldg(source + q);
                    words[4 * q] = v.x, words[4 * q + 1] = v.y, words[4 * q + 2] = v.z, words[4 * q + 3] = v.w;
                }
            } else {
#pragma unroll
                for (uint32_t q = 0; q < 16; ++q) words[q] = 0;
            }
#pragma unroll
            for (uint32_t i = 0; i < 16; ++i) {
                const float even = __uint_as_float(values[2 * i]) + __uint_as_float(words[i] << 16);
                const float odd = __uint_as_float(values[2 * i + 1]) + __uint_as_float(words[i] & 0xffff0000u);
                values[2 * i] = __float_as_uint(fmaxf(even, floor));
                values[2 * i + 1] = __float_as_uint(fmaxf(odd, floor));
            }
        }
    }
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i) {
        packed[i] = pack_bf16x2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
        packed[16 + i] = pack_bf16x2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
    }
}

// A unit of work of a cluster: an item and the run [k0, k1) of its k-blocks. Without a K split a
// unit is a whole item; with one, consecutive units are the runs of one item, so that they
// execute on different clusters at the same time.
struct Unit {
    Item item;
    uint32_t index;  // of the item
    uint32_t k0, k1;
};

template <bool kSplitK>
__device__ __forceinline__ uint32_t unit_count(const Schedule& plan) {
    return kSplitK ? plan.items * plan.splits : plan.items;
}

template <bool kSplitK>
__device__ __forceinline__ Unit unit_at(const Schedule& plan, uint32_t number) {
    Unit unit;
    if (kSplitK) {
        unit.index = number / plan.splits;
        unit.k0 = (number % plan.splits) * plan.split_blocks;
        const uint32_t stop = unit.k0 + plan.split_blocks;
        unit.k1 = stop < plan.k_blocks ? stop : plan.k_blocks;
    } else {
        unit.index = number;
        unit.k0 = 0;
        unit.k1 = plan.k_blocks;
    }
    unit.item = item_at(plan, unit.index);
    return unit;
}

// kAnyWidth: items may be 224 or 192 columns wide (Schedule::tile_n); without it the width is the
// constant 256 and the epilogue's passes are fixed at compile time, which is what launches of a
// few shallow items, whose epilogue is not hidden under a next item, are timed by.
template <bool kSplitK, bool kAnyWidth>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap a_map,
                          const __grid_constant__ CUtensorMap b_map,
                          const __grid_constant__ CUtensorMap c_map,
                          const __grid_constant__ CUtensorMap extra_map, const Schedule plan,
                          uint32_t* status) {
    // `extra_map`: the fp32 workspace's map in the K-split instantiation; in the one-launch one,
    // C's store map with a [32, 32] box for the last pass of items 224 or 160 columns wide.
    extern __shared__ __align__(1024) uint8_t dynamic_shared[];
    const uint32_t raw = smem_u32(dynamic_shared);
    const uint32_t base = raw;
    if (raw & (kBaseAlign - 1)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0u, static_cast<uint32_t>(kMisaligned));
        return;
    }

    const uint32_t a_ring = base + kPlan.a_ring.at;
    const uint32_t b_ring = base + kPlan.b_ring.at;
    const uint32_t bands = base + kPlan.bands.at;
    const uint32_t full = base + kPlan.full.at;
    const uint32_t empty = base + kPlan.empty.at;
    const uint32_t acc_full = base + kPlan.acc_full.at;
    const uint32_t acc_empty = base + kPlan.acc_empty.at;
    const uint32_t feed_full = base + kPlan.feed_full.at;
    const uint32_t feed_empty = base + kPlan.feed_empty.at;
    const uint32_t feed_go = base + kPlan.feed_go.at;
    const uint32_t claim_full = base + kPlan.claim_full.at;
    const uint32_t claim_answer = base + kPlan.claim_answer.at;
    const uint32_t feed_ring = base + kPlan.feed_ring.at;
    volatile uint32_t* feed_words = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.feed_ring.at);
    const uint32_t slot = base + kPlan.tmem_slot.at;
    const uint32_t stop_addr = base + kPlan.stop.at;
    volatile uint32_t* stop_flag =
        reinterpret_cast<volatile uint32_t*>(dynamic_shared + (stop_addr - raw));
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(dynamic_shared + (slot - raw));

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t peer = rank ^ 1u;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full + 8 * s, 1);
            mbar_init(empty + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 2 * kEpilogueWarps);
        for (uint32_t s = 0; s < kFeedSlots; ++s) {
            mbar_init(feed_full + 8 * s, 1);
            mbar_init(feed_empty + 8 * s, kFeedReaders);
        }
        mbar_init(feed_go, 1);
        mbar_init(claim_full, 1);
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

    // How a role learns its next unit of work. Static launches (no more units than resident
    // clusters, or a K split): cluster c walks units c, c + clusters, ... . Dynamic launches: the
    // role's next entry of the feed ring, which it hands back as soon as it has read it. `taken`
    // counts the role's reads, `previous` is the unit it read last; false = no further unit.
    const auto take = [&](uint32_t& taken, uint32_t previous, uint32_t& number, bool& live, bool whole_warp) -> bool {
        if (kSplitK || !plan.dynamic) {
            number = taken == 0 ? cluster_id_x() : previous + cluster_count_x();
            ++taken;
            return number < unit_count<kSplitK>(plan);
        }
        const uint32_t s = taken % kFeedSlots;
        if (!mbar_wait(feed_full + 8 * s, (taken / kFeedSlots) & 1u, site, kStallFeed, taken)) {
            live = false;
            return false;
        }
        fence_acq_rel_cluster();  // the entry was written from the leader CTA
        number = feed_words[s];
        if (whole_warp) __syncwarp();
        if (!whole_warp || lane == 0) mbar_arrive_cluster(mapa(feed_empty + 8 * s, 0));
        ++taken;
        return number != kNoItem;
    };

    if (warp == 0) {
        // ------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            uint32_t fill = 0, taken = 0, number = 0;
            bool live = true;
            while (live && take(taken, number, number, live, false)) {
                const Unit unit = unit_at<kSplitK>(plan, number);
                const Item& item = unit.item;
                if (item.halves == 0) continue;
                const int a_row = static_cast<int>(item.row + kBlockM * rank);
                // Each CTA stages its half of the item's columns: tile_n / 2 rows of B (the B map's box).
                const uint32_t tile_n = kAnyWidth ? plan.tile_n : kBlockN;
                const int b_row = static_cast<int>(item.column + (tile_n / 2) * rank);
                // Both CTAs' boxes land on the leader's barrier.
                const uint32_t pair_bytes = 2 * (item.halves * kATileBytes + (tile_n / 2) * kBlockK * 2);
                for (uint32_t k = unit.k0; k < unit.k1; ++k, ++fill) {
                    const uint32_t s = fill % kStages;
                    const uint32_t parity = (fill / kStages) & 1u;
                    if (!mbar_wait(empty + 8 * s, parity ^ 1u, site, kStallProducer, fill)) {
                        live = false;
                        break;
                    }
                    const uint32_t arrive_at = mapa(full + 8 * s, 0);
                    if (rank == 0) mbar_arrive_expect_tx(full + 8 * s, pair_bytes);
                    const int column = static_cast<int>(kBlockK * k);
                    tma_load_2d_pair(a_ring + (s * kHalves) * kATileBytes, &a_map, column, a_row,
                                     arrive_at);
                    tma_load_2d_pair(b_ring + s * kBTileBytes, &b_map, column, b_row, arrive_at);
                    if (item.halves == 2)
                        tma_load_2d_pair(a_ring + (s * kHalves + 1) * kATileBytes, &a_map, column,
                                         a_row + static_cast<int>(2 * kBlockM), arrive_at);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue (leader only)
        // One thread issues. An M256 N256 MMA occupies the pipe for 128 cycles, so the thread's
        // own cost per MMA does not show here (lane 0 or an elected lane: 1436 vs 1439 TFLOP/s).
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = plan.idesc;
            uint32_t drain = 0, count = 0, taken = 0, number = 0;
            bool live = true;
            while (live && take(taken, number, number, live, false)) {
                // The feed claims one item ahead: the next when this one begins.
                if (!kSplitK && plan.dynamic) mbar_arrive(feed_go);
                const Unit unit = unit_at<kSplitK>(plan, number);
                const Item& item = unit.item;
                if (item.halves == 0) continue;
                // The previous item's accumulators must have been read out.
                if (!mbar_wait(acc_empty, (count & 1u) ^ 1u, site, kStallMmaAccumulator, count)) {
                    live = false;
                    break;
                }
                tc_fence_after_sync();
                for (uint32_t k = unit.k0; k < unit.k1; ++k, ++drain) {
                    const uint32_t s = drain % kStages;
                    const uint32_t parity = (drain / kStages) & 1u;
                    if (!mbar_wait(full + 8 * s, parity, site, kStallMmaFull, drain)) {
                        live = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint64_t a0_desc = operand_descriptor(
                        a_ring + (s * kHalves) * kATileBytes, kKMajorLeadingBytes);
                    const uint64_t a1_desc = operand_descriptor(
                        a_ring + (s * kHalves + 1) * kATileBytes, kKMajorLeadingBytes);
                    const uint64_t b_desc =
                        operand_descriptor(b_ring + s * kBTileBytes, kKMajorLeadingBytes);
                    const uint32_t accumulate = k != unit.k0;
                    if (item.halves == 2) {
#pragma unroll
                        for (uint32_t chunk = 0; chunk < kBlockK / 16; ++chunk) {
                            // Advancing the 14-bit address field by 32 B per K=16 chunk.
                            const uint64_t step = (chunk * kKMajorChunkBytes) >> 4;
                            mma_ss<2>(tmem, a0_desc + step, b_desc + step, idesc, accumulate | chunk);
                            mma_ss<2>(tmem + kBlockN, a1_desc + step, b_desc + step, idesc,
                                      accumulate | chunk);
                        }
                    } else {
#pragma unroll
                        for (uint32_t chunk = 0; chunk < kBlockK / 16; ++chunk) {
                            const uint64_t step = (chunk * kKMajorChunkBytes) >> 4;
                            mma_ss<2>(tmem, a0_desc + step, b_desc + step, idesc, accumulate | chunk);
                        }
                    }
                    // The MMA's own retirement frees the stage, in both CTAs.
                    mma_commit<2>(empty + 8 * s);
                    mma_commit<2>(mapa(empty + 8 * s, 1));
                }
                if (!live) break;
                mma_commit<2>(acc_full);
                mma_commit<2>(mapa(acc_full, 1));
                ++count;
            }
        }
    } else if (warp == kFeedWarp) {
        // ------------------------------------------------ item feed (leader only, dynamic launches)
        if (!kSplitK && plan.dynamic && rank == 0 && lane == 0) {
            uint32_t published = 0, started = 0, claims = 0;
            bool live = true;
            // An entry goes to the same slot of both CTAs' rings, then each CTA's `feed_full`.
            const auto publish = [&](uint32_t value) {
                const uint32_t s = published % kFeedSlots;
                if (!mbar_wait(feed_empty + 8 * s, ((published / kFeedSlots) & 1u) ^ 1u, site, kStallFeed, published)) {
                    live = false;
                    return;
                }
                fence_acq_rel_cluster();  // the peer's readers are done with the slot
                feed_words[s] = value;
                st_shared_cluster_u32(mapa(feed_ring + 4 * s, 1), value);
                mbar_arrive(feed_full + 8 * s);
                mbar_arrive_cluster(mapa(feed_full + 8 * s, 1));
                ++published;
            };
            // This cluster's own item is the one the grid launched it for.
            publish(cluster_id_x());
            while (live) {
                // One item ahead and no more (a claimed item is this cluster's to do, however late):
                // the next claim goes out when the MMA thread begins the item published last.
                if (!mbar_wait(feed_go, started & 1u, site, kStallFeed, started)) break;
                ++started;
                mbar_arrive_expect_tx(claim_full, 16);
                clc_try_cancel(claim_answer, claim_full);
                if (!mbar_wait(claim_full, claims & 1u, site, kStallClaim, claims)) break;
                ++claims;
                uint32_t first_cta = 0;
                const bool granted = clc_query(claim_answer, first_cta);
                fence_proxy_async_shared();  // the answer is read before a later claim may overwrite it
                publish(granted ? first_cta / 2 : kNoItem);
                if (!granted) break;  // after a refusal no further request may be made
            }
        }
    } else {
        // ------------------------------------------------ epilogue (both CTAs)
        const uint32_t half = (warp - 2) >> 2;  // which accumulator this warp drains
        const uint32_t quadrant = warp & 3u;    // the tensor-memory lanes this warp may read
        const uint32_t band = bands + (warp - 2) * kBandBytes;
        const uint32_t t_row = tmem_address(tmem, 32 * quadrant, half * kBlockN);
        uint32_t count = 0, taken = 0, number = 0, upcoming = 0;
        bool live = true;
        // The unit after the current one is read as soon as the current one's accumulator is full:
        // whether there is one decides how the stores of the current one are staged.
        bool have = take(taken, 0, number, live, true), more = false;
        for (bool first = true;; first = false) {
            if (!first) number = upcoming, have = more;
            if (!live || !have) break;
            const Unit unit = unit_at<kSplitK>(plan, number);
            const Item& item = unit.item;
            if (item.halves == 0) {
                more = take(taken, number, upcoming, live, true);
                continue;
            }
            if (!mbar_wait(acc_full, count & 1u, site, kStallEpilogue, count)) {
                live = false;
                break;
            }
            ++count;
            tc_fence_after_sync();
            more = take(taken, number, upcoming, live, true);
            if (!live) break;
            const bool mine = half < item.halves;
            if constexpr (kSplitK) {
                // This unit's share of the sums: the warp's [32, 256] fp32 band goes into the workspace
                // 32 columns at a time through the staging tile and the copy engine's reduce-add.
                const int c_row =
                    static_cast<int>(item.row + 2 * kBlockM * half + kBlockM * rank + 32 * quadrant);
                if (mine) {
#pragma unroll 1
                    for (uint32_t pass = 0; pass < kBlockN / 32; ++pass) {
                        uint32_t v[32];
                        tmem_ld_32x32(t_row + 32 * pass, v);
                        tmem_wait_ld();
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
#pragma unroll
                        for (uint32_t chunk = 0; chunk < 8; ++chunk)
                            st_shared_v4(band + swizzled_chunk_offset(lane, chunk, 0), v[4 * chunk], v[4 * chunk + 1],
                                         v[4 * chunk + 2], v[4 * chunk + 3]);
                        fence_proxy_async_shared();
                        __syncwarp();
                        if (lane == 0) {
                            tma_reduce_add_2d(&extra_map, band, static_cast<int>(item.column + 32 * pass), c_row);
                            tma_store_commit();
                        }
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(mapa(acc_empty, 0));
                if (!mine) continue;
                // Count this unit in once its adds have been performed; the unit that completes the
                // count owns the band from here on.
                uint32_t* const counter = plan.arrivals + (unit.index * 2 + rank) * kEpilogueWarps + (warp - 2);
                uint32_t last = 0;
                if (lane == 0) {
                    tma_store_wait_all();
                    fence_proxy_async_global();  // the adds went through the async proxy, the reads below will not
                    __threadfence();
                    last = atomicAdd(counter, 1u) + 1u == plan.splits ? 1u : 0u;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (!last) continue;
                __threadfence();
                fence_proxy_async_global();
                // Read the sums back (through the L2, where the adds were made), finish them as the
                // one-launch epilogue does, and leave the workspace as it was found: zero.
                float* const sums = plan.partial + static_cast<size_t>(c_row + lane) * plan.n + item.column;
#pragma unroll 1
                for (uint32_t pass = 0; pass < kPasses; ++pass) {
                    uint32_t lo[32], hi[32], packed[32];
                    float4* const source = reinterpret_cast<float4*>(sums + pass * kStageColumns);
#pragma unroll
                    for (uint32_t q = 0; q < 8; ++q) {
                        const float4 x = __ldcg(source + q), y = __ldcg(source + 8 + q);
                        lo[4 * q] = __float_as_uint(x.x), lo[4 * q + 1] = __float_as_uint(x.y);
                        lo[4 * q + 2] = __float_as_uint(x.z), lo[4 * q + 3] = __float_as_uint(x.w);
                        hi[4 * q] = __float_as_uint(y.x), hi[4 * q + 1] = __float_as_uint(y.y);
                        hi[4 * q + 2] = __float_as_uint(y.z), hi[4 * q + 3] = __float_as_uint(y.w);
                    }
#pragma unroll
                    for (uint32_t q = 0; q < 16; ++q) __stcg(source + q, make_float4(0.0f, 0.0f, 0.0f, 0.0f));
                    finish_pass(lo, hi, plan, item.column + pass * kStageColumns, packed);
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
#pragma unroll
                    for (uint32_t chunk = 0; chunk < 8; ++chunk)
                        st_shared_v4(band + swizzled_chunk_offset(lane, chunk, 0), packed[4 * chunk],
                                     packed[4 * chunk + 1], packed[4 * chunk + 2], packed[4 * chunk + 3]);
                    fence_proxy_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        if (plan.accumulate)
                            tma_reduce_add_2d(&c_map, band, static_cast<int>(item.column + pass * kStageColumns), c_row);
                        else
                            tma_store_2d(&c_map, band, static_cast<int>(item.column + pass * kStageColumns), c_row);
                        tma_store_commit();
                    }
                }
                if (lane == 0) *counter = 0;
                continue;
            }
            // Read this warp's band of the item out as bf16 pairs, then release the accumulator: the
            // stores below overlap the next item's main loop. An item is 256, 224 or 192 columns wide:
            // three passes of 64 columns, then a fourth of 64, of 32 (`kLastNarrow`) or none.
            const uint32_t last_pass = !kAnyWidth || plan.tile_n == kBlockN ? kLastWhole
                                       : plan.tile_n == kBlockN - 32        ? kLastNarrow
                                                                            : kLastNone;
            uint32_t held[kPasses][32];
            if (mine) {
#pragma unroll
                for (uint32_t pass = 0; pass < kPasses; ++pass) {
                    uint32_t lo[32], hi[32];
                    if (pass + 1 < kPasses || last_pass == kLastWhole) {
                        tmem_ld_32x32(t_row + pass * kStageColumns, lo);
                        tmem_ld_32x32(t_row + pass * kStageColumns + 32, hi);
                        tmem_wait_ld();
                        finish_pass(lo, hi, plan, item.column + pass * kStageColumns, held[pass]);
                    } else if (last_pass == kLastNarrow) {
                        tmem_ld_32x32(t_row + pass * kStageColumns, lo);
                        tmem_wait_ld();
                        finish_pass(lo, lo, plan, item.column + pass * kStageColumns, held[pass], 1);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa(acc_empty, 0));
            if (!mine) continue;

            const int c_row =
                static_cast<int>(item.row + 2 * kBlockM * half + kBlockM * rank + 32 * quadrant);
            // A 64-column pass of this lane's row into a [32, 64] SWIZZLE_128B staging tile.
            const auto stage = [&](uint32_t tile, const uint32_t (&words)[32]) {
#pragma unroll
                for (uint32_t chunk = 0; chunk < 8; ++chunk)
                    st_shared_v4(tile + swizzled_chunk_offset(lane, chunk, 0), words[4 * chunk], words[4 * chunk + 1],
                                 words[4 * chunk + 2], words[4 * chunk + 3]);
            };
            // The 32-column pass: dense rows of 64 bytes (the narrow store map is not swizzled).
            const auto stage_narrow = [&](uint32_t tile, const uint32_t (&words)[32]) {
#pragma unroll
                for (uint32_t chunk = 0; chunk < 4; ++chunk)
                    st_shared_v4(tile + 64 * lane + 16 * chunk, words[4 * chunk], words[4 * chunk + 1],
                                 words[4 * chunk + 2], words[4 * chunk + 3]);
            };
            // One thread: a staged pass to C (the 32-column pass through the narrow store map, which
            // this instantiation receives in place of the workspace's).
            const auto store = [&](const CUtensorMap* map, uint32_t tile, uint32_t pass) {
                const int column = static_cast<int>(item.column + pass * kStageColumns);
                if (plan.accumulate)
                    tma_reduce_add_2d(map, tile, column, c_row);
                else
                    tma_store_2d(map, tile, column, c_row);
            };
            if (!more) {
                // This CTA's last item: no load is outstanding or to come and every MMA that read
                // the operand ring has retired (acc_full), so the ring is free shared memory. Each
                // warp stages all its passes there at once, kPasses tiles of its own, and the
                // stores go out back to back instead of waiting for one staging tile in turn.
                const uint32_t spare = a_ring + (warp - 2) * kPasses * kBandBytes;
#pragma unroll
                for (uint32_t pass = 0; pass < kPasses; ++pass) {
                    const bool narrow = pass + 1 == kPasses && last_pass == kLastNarrow;
                    if (pass + 1 == kPasses && last_pass == kLastNone) break;
                    // Staged and sent pass by pass: the copy engine reads one tile while the next is staged.
                    if (narrow)
                        stage_narrow(spare + pass * kBandBytes, held[pass]);
                    else
                        stage(spare + pass * kBandBytes, held[pass]);
                    fence_proxy_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        store(narrow ? &extra_map : &c_map, spare + pass * kBandBytes, pass);
                        tma_store_commit();
                    }
                }
                continue;
            }
#pragma unroll
            for (uint32_t pass = 0; pass < kPasses; ++pass) {
                if (pass + 1 == kPasses && last_pass == kLastNone) break;
                // The store that last read this warp's staging tile must be done reading it.
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
                if (pass + 1 == kPasses && last_pass == kLastNarrow)
                    stage_narrow(band, held[pass]);
                else
                    stage(band, held[pass]);
                // Every writer publishes to the async proxy, then one lane stores.
                fence_proxy_async_shared();
                __syncwarp();
                if (lane == 0) {
                    if (pass + 1 == kPasses && last_pass == kLastNarrow)
                        store(&extra_map, band, pass);
                    else
                        store(&c_map, band, pass);
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_before_exit();
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

// ------------------------------------------------------------------ the narrow tile
//
// Launches of a few wide items leave most SMs idle, and when K is shallow too the wide kernel's
// fixed cost (cluster rendezvous, a 4 x 48 KiB ring that is latency-bound on 16 clusters, a serial
// [128, 256] epilogue per CTA) is most of the launch. The reference meets such launches with a
// narrow cluster tile (`gemm_sol_m256_n128`, examples/src/gemm_sol.rs:1063, dispatch :1335-1337);
// here they get one CTA per [128, 128] tile of C, no cluster, cta_group::1 MMAs (M128 N128 K16),
// three 32 KiB stages and 128 tensor-memory columns, so that two CTAs share an SM and one's
// epilogue runs under the other's main loop. Same operand maps, same C map, same fused epilogue.
namespace narrow {

constexpr uint32_t kTile = 128;     // rows and columns of C per CTA
// Three stages let two CTAs share an SM, which a grid of more tiles than SMs wants (one's epilogue
// under the other's main loop); a grid of fewer tiles leaves every CTA alone on its SM, where three
// 32 KiB stages are too few bytes in flight to cover the L2's latency, and takes six.
constexpr uint32_t kStagesShared = 3;
constexpr uint32_t kStagesAlone = 6;
constexpr uint32_t kEpilogueWarps = 4;
constexpr uint32_t kThreads = (2 + kEpilogueWarps) * 32;
constexpr uint32_t kTileBytes = kTile * kBlockK * 2;  // one [128, 64] operand tile
constexpr uint32_t kTmemColumns = kTile;
// K split across a cluster: the CTAs of a cluster take consecutive runs of one tile's k-blocks and
// the others hand their fp32 tiles to the first through distributed shared memory, into its
// operand ring, which is idle by then: one [128, 128] fp32 tile, 64 KiB, per contributor.
constexpr uint32_t kMaxSlices = 4;
constexpr uint32_t kPartialBytes = kTile * kTile * 4;
static_assert((kMaxSlices - 1) * kPartialBytes <= 2 * kStagesAlone * kTileBytes, "the partial tiles must fit the ring");

template <uint32_t kStages>
struct Plan {
    SharedPlan a_ring, b_ring, bands, full, empty, acc_full, go, partial_full, tmem_slot, stop, end;
    constexpr Plan()
        : a_ring(SharedPlan{}.tile_ring(kTile, kBlockK, 2, kStages)),
          b_ring(a_ring.tile_ring(kTile, kBlockK, 2, kStages)),
          // one staging tile per epilogue warp and pass where the shared memory allows (a CTA alone on its
          // SM): the second pass is then staged while the copy engine still reads the first
          bands(b_ring.tile_ring(32, kStageColumns, 2, kEpilogueWarps * (kStages == kStagesAlone ? kTile / kStageColumns : 1))),
          full(bands.semaphores(kStages)),
          empty(full.semaphores(kStages)),
          acc_full(empty.semaphore()),
          go(acc_full.semaphore()),
          partial_full(go.semaphore()),
          tmem_slot(partial_full.tmem_slot()),
          stop(tmem_slot.word()),
          end(stop) {}
};
template <uint32_t kStages>
constexpr uint32_t shared_bytes() {
    return static_cast<uint32_t>(Plan<kStages>{}.end.bytes());
}
// Two CTAs per SM: each pays about 1 KiB of reserved shared memory on top of its plan.
static_assert(2 * (shared_bytes<kStagesShared>() + 1024) <= 233472, "two narrow CTAs must fit one SM's shared memory");
static_assert(shared_bytes<kStagesAlone>() <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");

// Byte offset of 16-byte chunk `chunk` (0..31) of row `row` inside a partial tile: the chunk index
// is folded with the row so that the eight lanes of a quarter-warp touch eight different bank groups.
__device__ __forceinline__ uint32_t partial_offset(uint32_t row, uint32_t chunk) {
    return row * (kTile * 4) + (((chunk ^ row) & 31u) << 4);
}

template <uint32_t kStages, bool kSliced>
__global__ void __launch_bounds__(kThreads, kStages == kStagesShared ? 2 : 1)
    gemm_bf16_narrow_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map,
                            const __grid_constant__ CUtensorMap c_map, const Schedule plan, uint32_t* status) {
    constexpr Plan<kStages> kPlan{};
    static_assert(kPlan.a_ring.at % 1024 == 0 && kPlan.b_ring.at % 1024 == 0 && kPlan.bands.at % 1024 == 0,
                  "swizzled tiles must start on a 1024-byte boundary");
    extern __shared__ __align__(1024) uint8_t dynamic_shared[];
    const uint32_t base = smem_u32(dynamic_shared);
    if (base & (kBaseAlign - 1)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0u, static_cast<uint32_t>(kMisaligned));
        return;
    }
    const uint32_t a_ring = base + kPlan.a_ring.at;
    const uint32_t b_ring = base + kPlan.b_ring.at;
    const uint32_t bands = base + kPlan.bands.at;
    const uint32_t full = base + kPlan.full.at;
    const uint32_t empty = base + kPlan.empty.at;
    const uint32_t acc_full = base + kPlan.acc_full.at;
    const uint32_t go = base + kPlan.go.at;
    const uint32_t partial_full = base + kPlan.partial_full.at;
    const uint32_t slot = base + kPlan.tmem_slot.at;
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.stop.at);
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.tmem_slot.at);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row0 = kTile * blockIdx.y;
    const uint32_t column0 = kTile * blockIdx.x;
    // This CTA's run of k-blocks: all of them, or its slice of the cluster's.
    const uint32_t slices = kSliced ? gridDim.z : 1u;
    const uint32_t slice = kSliced ? cluster_ctarank() : 0u;
    const uint32_t run = (plan.k_blocks + slices - 1) / slices;
    const uint32_t k0 = slice * run;
    const uint32_t k1 = k0 + run < plan.k_blocks ? k0 + run : plan.k_blocks;
    uint32_t preloaded = 0;  // k-blocks whose loads the producer thread issued before the rendezvous

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full + 8 * s, 1);
            mbar_init(empty + 8 * s, 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(go, 1);
        mbar_init(partial_full, 1);
        *stop_flag = 0;
        fence_mbarrier_init();
        fence_proxy_async_shared();
        // This thread is the producer, and the ring's first stages are free by construction: their
        // loads go out now, under the tensor-memory allocation and the rendezvous below (a launch of
        // a few k-blocks is mostly its own start-up).
        preloaded = k1 - k0 < kStages ? k1 - k0 : kStages;
        for (uint32_t i = 0; i < preloaded; ++i) {
            mbar_arrive_expect_tx(full + 8 * i, 2 * kTileBytes);
            const int column = static_cast<int>(kBlockK * (k0 + i));
            tma_load_2d(a_ring + i * kTileBytes, &a_map, column, static_cast<int>(row0), full + 8 * i);
            tma_load_2d(b_ring + i * kTileBytes, &b_map, column, static_cast<int>(column0), full + 8 * i);
        }
        prefetch_tensormap(&c_map);
    }
    if (warp == 1) {
        tmem_alloc<1>(slot, kTmemColumns);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (kSliced) cluster_sync();  // every CTA's barriers exist before a peer arrives on them
    tc_fence_after_sync();
    const uint32_t tmem = *slot_ptr;
    const StallSite site{status, stop_flag, 0};
    // A k-block is four MMAs, 256 tensor cycles: a thread suspended in try_wait wakes later than
    // that, so the two roles on the operand ring poll instead.
    const StallSite prompt{status, stop_flag, 0, kWaitBudgetCycles, true};

    if (warp == 0) {
        // ------------------------------------------------ producer
        if (lane == 0) {
            for (uint32_t k = k0 + preloaded; k < k1; ++k) {
                const uint32_t s = (k - k0) % kStages;
                if (!mbar_wait(empty + 8 * s, (((k - k0) / kStages) & 1u) ^ 1u, prompt, kStallProducer, k)) break;
                mbar_arrive_expect_tx(full + 8 * s, 2 * kTileBytes);
                const int column = static_cast<int>(kBlockK * k);
                tma_load_2d(a_ring + s * kTileBytes, &a_map, column, static_cast<int>(row0), full + 8 * s);
                tma_load_2d(b_ring + s * kTileBytes, &b_map, column, static_cast<int>(column0), full + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issue
        // One elected thread (see the note at elect_one: the tight issue sequence matters when an
        // MMA is 64 cycles of the pipe).
        if (elect_one()) {
            bool live = true;
            for (uint32_t k = k0; k < k1; ++k) {
                const uint32_t s = (k - k0) % kStages;
                if (!mbar_wait(full + 8 * s, ((k - k0) / kStages) & 1u, prompt, kStallMmaFull, k)) {
                    live = false;
                    break;
                }
                tc_fence_after_sync();
                const uint64_t a_desc = operand_descriptor(a_ring + s * kTileBytes, kKMajorLeadingBytes);
                const uint64_t b_desc = operand_descriptor(b_ring + s * kTileBytes, kKMajorLeadingBytes);
#pragma unroll
                for (uint32_t chunk = 0; chunk < kBlockK / 16; ++chunk) {
                    const uint64_t step = (chunk * kKMajorChunkBytes) >> 4;
                    mma_ss<1>(tmem, a_desc + step, b_desc + step, plan.idesc, (k != k0) | chunk);
                }
                mma_commit<1>(empty + 8 * s);
            }
            if (live) mma_commit<1>(acc_full);
        }
    } else {
        // ------------------------------------------------ epilogue: one 32-row band per warp
        const uint32_t quadrant = warp & 3u;
        const uint32_t band = bands + (warp - 2) * kBandBytes;
        const uint32_t t_row = tmem_address(tmem, 32 * quadrant, 0);
        bool live = mbar_wait(acc_full, 0, site, kStallEpilogue, 0);
        if (live) tc_fence_after_sync();
        const uint32_t row = 32 * quadrant + lane;  // of the tile
        if (kSliced && live && slice != 0) {
            // A contributor: this warp's 32 rows of the fp32 tile are staged in the CTA's own ring
            // (idle: its MMAs have retired) and, once the first CTA's ring is idle too (`go`), go
            // into this CTA's slot there as one 16 KiB bulk copy that completes on the first CTA's
            // `partial_full`. (Written there by 4096 remote 16-byte stores instead, the hand-over
            // took several microseconds.)
#pragma unroll 1
            for (uint32_t part = 0; part < kTile / 32; ++part) {
                uint32_t v[32];
                tmem_ld_32x32(t_row + 32 * part, v);
                tmem_wait_ld();
#pragma unroll
                for (uint32_t chunk = 0; chunk < 8; ++chunk)
                    st_shared_v4(a_ring + partial_offset(row, 8 * part + chunk), v[4 * chunk], v[4 * chunk + 1],
                                 v[4 * chunk + 2], v[4 * chunk + 3]);
            }
            fence_proxy_async_shared();
            __syncwarp();
            live = mbar_wait(go, 0, site, kStallEpilogue, 1);
            if (live && lane == 0) {
                constexpr uint32_t kBandOfPartial = 32 * kTile * 4;
                const uint32_t band_at = quadrant * kBandOfPartial;
                bulk_copy_to_peer(mapa(a_ring + (slice - 1) * kPartialBytes + band_at, 0), a_ring + band_at, kBandOfPartial,
                                  mapa(partial_full, 0));
            }
        } else if (live) {
            if (kSliced) {
                // The first CTA: its MMAs have retired, so its ring is free for the others' tiles.
                if (warp == 2 && lane == 0) {
                    mbar_arrive_expect_tx(partial_full, (slices - 1) * kPartialBytes);
                    for (uint32_t peer = 1; peer < slices; ++peer) mbar_arrive_cluster(mapa(go, peer));
                }
                live = mbar_wait(partial_full, 0, site, kStallEpilogue, 2);
            }
            const int c_row = static_cast<int>(row0 + 32 * quadrant);
#pragma unroll 1
            for (uint32_t pass = 0; live && pass < kTile / kStageColumns; ++pass) {
                uint32_t lo[32], hi[32], packed[32];
                tmem_ld_32x32(t_row + pass * kStageColumns, lo);
                tmem_ld_32x32(t_row + pass * kStageColumns + 32, hi);
                tmem_wait_ld();
                if (kSliced) {
                    for (uint32_t peer = 1; peer < slices; ++peer) {
                        const uint32_t slot_base = a_ring + (peer - 1) * kPartialBytes;
#pragma unroll
                        for (uint32_t chunk = 0; chunk < 8; ++chunk) {
                            uint32_t x[4], y[4];
                            ld_shared_v4(slot_base + partial_offset(row, 16 * pass + chunk), x);
                            ld_shared_v4(slot_base + partial_offset(row, 16 * pass + 8 + chunk), y);
#pragma unroll
                            for (uint32_t i = 0; i < 4; ++i) {
                                lo[4 * chunk + i] = __float_as_uint(__uint_as_float(lo[4 * chunk + i]) + __uint_as_float(x[i]));
                                hi[4 * chunk + i] = __float_as_uint(__uint_as_float(hi[4 * chunk + i]) + __uint_as_float(y[i]));
                            }
                        }
                    }
                }
                finish_pass(lo, hi, plan, column0 + pass * kStageColumns, packed);
                // A tile of its own per pass, or the one tile once the store that read it last is done reading.
                constexpr bool kTilePerPass = kStages == kStagesAlone;
                const uint32_t tile = kTilePerPass ? band + pass * kEpilogueWarps * kBandBytes : band;
                if (!kTilePerPass) {
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                }
#pragma unroll
                for (uint32_t chunk = 0; chunk < 8; ++chunk)
                    st_shared_v4(tile + swizzled_chunk_offset(lane, chunk, 0), packed[4 * chunk], packed[4 * chunk + 1],
                                 packed[4 * chunk + 2], packed[4 * chunk + 3]);
                fence_proxy_async_shared();
                __syncwarp();
                if (lane == 0) {
                    const int column = static_cast<int>(column0 + pass * kStageColumns);
                    if (plan.accumulate)
                        tma_reduce_add_2d(&c_map, tile, column, c_row);
                    else
                        tma_store_2d(&c_map, tile, column, c_row);
                    tma_store_commit();
                }
            }
            if (lane == 0) tma_store_wait_before_exit();
        }
    }

    // ---------------------------------------------------- teardown
    if (*stop_flag) {
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (kSliced) cluster_sync();  // no CTA leaves while a peer may still write into it or arrive on it
    if (warp == 1) tmem_dealloc<1>(tmem, kTmemColumns);
}

}  // namespace narrow

// The item list of a launch over `clusters` resident clusters: whole [512, 256]
// tiles, with the last partial wave re-cut into single halves when it holds at
// most half a wave of tiles (two short half-waves then beat one long one).
static Schedule schedule(uint32_t m, uint32_t n, uint32_t k, uint32_t group, uint32_t clusters,
                         uint32_t flags = 0, uint32_t tile_n = kBlockN) {
    Schedule plan;
    plan.idesc = instruction_descriptor(2 * kBlockM, tile_n, false, false,
                                        (flags & FK_GEMM_F16_OPERANDS) ? 0u : 1u);
    plan.tile_n = tile_n;
    plan.dynamic = 0;
    plan.accumulate = (flags & FK_GEMM_ACCUMULATE) ? 1u : 0u;
    plan.relu = (flags & FK_GEMM_RELU) ? 1u : 0u;
    plan.bias = nullptr;
    plan.splits = 1;
    plan.split_blocks = k / kBlockK;
    plan.n = n;
    plan.partial = nullptr;
    plan.arrivals = nullptr;
    plan.m = m;
    plan.tiles_m = (m + kHalves * 2 * kBlockM - 1) / (kHalves * 2 * kBlockM);
    plan.tiles_n = n / tile_n;
    // A width at or past the tile rows is already the column-major walk; clamping keeps
    // `group * columns` inside 32 bits whatever the caller passes.
    plan.group = group < plan.tiles_m ? group : plan.tiles_m;
    plan.k_blocks = k / kBlockK;
    const uint32_t tiles = plan.tiles_m * plan.tiles_n;
    const uint32_t tail = tiles % clusters;
    const bool recut = tail != 0 && 2 * tail <= clusters;
    plan.whole = recut ? tiles - tail : tiles;
    plan.items = plan.whole + kHalves * (tiles - plan.whole);
    return plan;
}

// Time of a launch in units of one cluster walking K over 32 columns of a two-half item: whole
// waves, and a last one that costs half when `schedule` re-cuts it.
static uint32_t wave_cost(const Schedule& plan, uint32_t clusters) {
    const uint32_t tiles = plan.tiles_m * plan.tiles_n;
    const uint32_t tail = tiles % clusters;
    const uint32_t half_waves = 2 * (tiles / clusters) + (tail == 0 ? 0u : plan.whole != tiles ? 1u : 2u);
    return half_waves * (plan.tile_n / 32);
}

// Columns per item for a launch of the wide kernel whose maps this library builds. A tile count just
// past a whole number of waves wastes most of its last wave: 8192 x 3584 (an eighth of the 28672-column
// up-projection) is 224 items of [512, 256] = 3 waves of 74 and 2 items, 3.5 wave-times even re-cut,
// but 256 items of [512, 224] = 3 waves and 34, which re-cut into 68 halves fill half a wave:
// 3.5 x 224 / 256 = 3.06. Measured on B200 (back-to-back launches at the power limit, 256 / 224 wide):
// 8192 x 3584 x 8192: 364 / 343 us; 2048 x 5376 x 4096: 107 / 95; but 8192 x 7168 x 8192 (6.5 wave-times
// against 6.125): 704 / 720, and 8192 x 28672 x 8192 (24.5 both): 2822 / 2873 -- the narrower item costs
// about 2 % per flop (A re-read more often, more items to drain), and at the power limit a thin last
// wave is partly repaid in clock by the SMs that idle through it. So narrower items must promise 10 %.
static uint32_t choose_tile_n(uint32_t m, uint32_t n, uint32_t k, uint32_t clusters) {
    uint32_t best = kBlockN;
    uint32_t best_cost = wave_cost(schedule(m, n, k, 1, clusters, 0, kBlockN), clusters);
    for (uint32_t tile_n = kBlockN - 32; tile_n >= kBlockN - 64; tile_n -= 32) {
        if (n % tile_n) continue;
        const uint32_t cost = wave_cost(schedule(m, n, k, 1, clusters, 0, tile_n), clusters);
        if (100ull * cost < 90ull * best_cost) best = tile_n, best_cost = cost;
    }
    return best;
}

}  // namespace gemm
}  // namespace fk

// ------------------------------------------------------------------ C ABI

using namespace fk;

extern "C" uint32_t fk_gemm_shared_bytes(void) { return gemm::kSharedBytes; }
extern "C" uint32_t fk_gemm_threads(void) { return gemm::kThreads; }

extern "C" uint32_t fk_gemm_grid(uint32_t m, uint32_t n, uint32_t sm_count) {
    const uint32_t clusters = sm_count / 2;
    if (clusters == 0) return 0;
    const gemm::Schedule plan = gemm::schedule(m, n, gemm::kBlockK, 1, clusters);
    return 2 * (plan.items < clusters ? plan.items : clusters);
}

// Which launches take the narrow tile when the caller does not say. Measured on B200 (device time per
// launch from CUDA-graph replays, wide / narrow, microseconds): 1024 x 1024 x 512: 8.4 / 5.5;
// 1024 x 1024 x 4096: 25.5 / 17.2; 2048 x 1024 x 8192: 46.4 / 31.1; 2048 x 2048 x 256: 7.6 / 5.7;
// 2048 x 2048 x 1024: 11.5 / 10.0; 2048 x 2048 x 2048: 16.5 / 16.1; 2048 x 2048 x 4096: 26.4 / 29.9;
// 4096 x 2048 x 512: 12.9 / 12.4; 3072 x 3072 x 1024: 20.1 / 19.9; 4096 x 4096 x 256: 14.5 / 17.9.
// So: up to 128 narrow tiles at any depth (the wide items would leave most SMs idle), up to two
// CTAs per SM's worth while K is at most 2048 (past that the wide tile's operand reuse wins).
static bool narrow_by_default(uint32_t m, uint32_t n, uint32_t k, uint32_t sm_count) {
    const uint64_t tiles = uint64_t(m / gemm::narrow::kTile) * (n / gemm::narrow::kTile);
    if (tiles <= 128) return true;
    return tiles <= 2ull * sm_count && k <= 2048;
}

static bool takes_narrow(uint32_t m, uint32_t n, uint32_t k, uint32_t flags, uint32_t sm_count) {
    return (flags & FK_GEMM_TILE_NARROW) || (!(flags & FK_GEMM_TILE_WIDE) && narrow_by_default(m, n, k, sm_count));
}

// Clusters of `slices` CTAs of the sliced narrow kernel this device holds at once (0 if the runtime
// cannot say), asked once per device and size.
static uint32_t resident_narrow_clusters(uint32_t slices) {
    static std::mutex guard;
    static int known[64][gemm::narrow::kMaxSlices + 1];  // 0 = not asked yet, -1 = no answer
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64 || slices > gemm::narrow::kMaxSlices) return 0;
    std::lock_guard<std::mutex> lock(guard);
    if (known[device][slices] == 0) {
        const auto kernel = gemm::narrow::gemm_bf16_narrow_kernel<gemm::narrow::kStagesAlone, true>;
        const uint32_t bytes = gemm::narrow::shared_bytes<gemm::narrow::kStagesAlone>();
        uint32_t limit = 0;
        int clusters = 0;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(1, 1, slices);
        config.blockDim = dim3(gemm::narrow::kThreads, 1, 1);
        config.dynamicSmemBytes = bytes;
        cudaLaunchAttribute cluster;
        cluster.id = cudaLaunchAttributeClusterDimension;
        cluster.val.clusterDim.x = 1, cluster.val.clusterDim.y = 1, cluster.val.clusterDim.z = slices;
        config.attrs = &cluster;
        config.numAttrs = 1;
        if (fk_admit_shared_plan(reinterpret_cast<const void*>(kernel), bytes, &limit) == FK_OK &&
            cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) == cudaSuccess && clusters > 0)
            known[device][slices] = clusters;
        else
            known[device][slices] = -1, (void)cudaGetLastError();
    }
    return known[device][slices] > 0 ? static_cast<uint32_t>(known[device][slices]) : 0u;
}

// The launch behind every GEMM entry. `tile_n` is the width of the wide kernel's items: 256 with the
// caller's maps (B's box is then 128 rows); the entries that build the maps themselves may pass 224
// or 192 with a B box of tile_n / 2 rows and, when tile_n is an odd multiple of 32, `c_narrow_map`,
// C's store map with a [32, 32] box (otherwise unused: any valid map).
static int launch_fused(const void* a_map, const void* b_map, const void* c_map, const void* c_narrow_map,
                        uint32_t tile_n, const void* bias, uint32_t m, uint32_t n, uint32_t k, uint32_t group,
                        uint32_t flags, void* stream, uint32_t* device_status) {
    if (flags & ~(FK_GEMM_F16_OPERANDS | FK_GEMM_ACCUMULATE | FK_GEMM_RELU | FK_GEMM_TILE_NARROW | FK_GEMM_TILE_WIDE |
                  FK_GEMM_ORDER_FEED | FK_GEMM_ORDER_STATIC))
        return fk_fail(FK_ERR_INVALID, "unknown GEMM flags 0x%x", flags);
    if ((flags & FK_GEMM_TILE_NARROW) && (flags & FK_GEMM_TILE_WIDE))
        return fk_fail(FK_ERR_INVALID, "the narrow and the wide tile were both asked for");
    if ((flags & FK_GEMM_ORDER_FEED) && (flags & FK_GEMM_ORDER_STATIC))
        return fk_fail(FK_ERR_INVALID, "the fed and the static item order were both asked for");
    if (reinterpret_cast<uintptr_t>(bias) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "the bias vector wants 16-byte alignment");
    if (!a_map || !b_map || !c_map) return fk_fail(FK_ERR_INVALID, "a tensor map pointer is null");
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN ||
        k % gemm::kBlockK)
        return fk_fail(FK_ERR_SHAPE, "%ux%ux%u does not divide the %ux%ux%u tiling", m, n, k,
                       2 * gemm::kBlockM, gemm::kBlockN, gemm::kBlockK);
    if (group == 0)
        return fk_fail(FK_ERR_SHAPE, "a traversal group width of 0 has no tiles in it");

    DeviceFacts facts;
    const int known = device_facts(&facts);
    if (known != FK_OK) return known;
    const int sm_count = facts.sm_count;
    uint32_t limit = 0;
    const int admitted = fk_admit_shared_plan(
        reinterpret_cast<const void*>(gemm::gemm_bf16_pair_kernel<false, false>), gemm::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;

    const uint32_t clusters = static_cast<uint32_t>(sm_count) / 2;
    const bool narrow = takes_narrow(m, n, k, flags, static_cast<uint32_t>(sm_count));
    gemm::Schedule plan = gemm::schedule(m, n, k, group, clusters, flags, narrow ? gemm::kBlockN : tile_n);
    plan.bias = static_cast<const uint16_t*>(bias);
    if (narrow) {
        // One CTA per [128, 128] tile; the A and B maps' boxes are [64, 128] already, C's [64, 32].
        plan.idesc = instruction_descriptor(gemm::narrow::kTile, gemm::narrow::kTile, false, false,
                                            (flags & FK_GEMM_F16_OPERANDS) ? 0u : 1u);
        const dim3 tiles(n / gemm::narrow::kTile, m / gemm::narrow::kTile, 1);
        if (tiles.y > 65535) return fk_fail(FK_ERR_SHAPE, "%u rows is past what the narrow tile's grid takes", m);
        const auto launch_narrow = [&](auto kernel, uint32_t bytes, uint32_t slices) -> int {
            const int narrow_admitted = fk_admit_shared_plan(reinterpret_cast<const void*>(kernel), bytes, &limit);
            if (narrow_admitted != FK_OK) return narrow_admitted;
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(tiles.x, tiles.y, slices);
            config.blockDim = dim3(gemm::narrow::kThreads, 1, 1);
            config.dynamicSmemBytes = bytes;
            config.stream = static_cast<cudaStream_t>(stream);
            cudaLaunchAttribute cluster;
            cluster.id = cudaLaunchAttributeClusterDimension;
            cluster.val.clusterDim.x = 1, cluster.val.clusterDim.y = 1, cluster.val.clusterDim.z = slices;
            config.attrs = &cluster;
            config.numAttrs = slices > 1 ? 1 : 0;
            FK_CUDA(cudaLaunchKernelEx(&config, kernel, *static_cast<const CUtensorMap*>(a_map),
                                       *static_cast<const CUtensorMap*>(b_map), *static_cast<const CUtensorMap*>(c_map),
                                       plan, device_status));
            return FK_OK;
        };
        const uint64_t count = uint64_t(tiles.x) * tiles.y;
        // Few tiles and a deep K: a cluster per tile, each CTA a run of the k-blocks. The hand-over
        // (two cluster rendezvous, 64 KiB per contributor staged and bulk-copied into the first CTA's
        // shared memory, the first CTA summing them) costs 2-3 us, a k-block on a lone CTA ~0.21 us:
        // worth it from 64 k-blocks on, in runs of at least 16 (1024 x 1024 x 4096: 16.4 -> 14.9 us;
        // 256 x 256 x 4096: 16.2 -> 12.9; 512 x 512 x 16384: 56 -> 23; but 1024 x 1024 x 2048 in two runs
        // of 16: 10.0 -> 11.5) -- and only while every cluster is resident at once: clusters of four
        // pack a GPC's SMs worse than single CTAs (768 x 768 x 4096, 36 clusters of four: two rounds,
        // 25.6 us against 16.4 uncut), so the count is the runtime's, not SMs / slices.
        uint32_t slices = 1;
        while (plan.k_blocks >= 64 && slices < gemm::narrow::kMaxSlices && plan.k_blocks / (2 * slices) >= 16 &&
               count <= resident_narrow_clusters(2 * slices))
            slices *= 2;
        if (slices > 1)
            return launch_narrow(gemm::narrow::gemm_bf16_narrow_kernel<gemm::narrow::kStagesAlone, true>,
                                 gemm::narrow::shared_bytes<gemm::narrow::kStagesAlone>(), slices);
        if (count <= static_cast<uint64_t>(sm_count))
            return launch_narrow(gemm::narrow::gemm_bf16_narrow_kernel<gemm::narrow::kStagesAlone, false>,
                                 gemm::narrow::shared_bytes<gemm::narrow::kStagesAlone>(), 1);
        return launch_narrow(gemm::narrow::gemm_bf16_narrow_kernel<gemm::narrow::kStagesShared, false>,
                             gemm::narrow::shared_bytes<gemm::narrow::kStagesShared>(), 1);
    }
    // Long launches: one cluster per item in the grid, handed out as clusters fall free (the resident
    // ones never exit before the grid is used up). What that order buys is that clusters cannot drift
    // waves apart, which takes several waves to matter; and the feed learns the next item a claim's
    // round trip (~2 us) after the current one begins, which the producer of a short item would wait
    // out at every item boundary (4096 x 4096 x 512, 128 items of 8 k-blocks: 23.9 us against 19.4
    // with the static walk). So: from four waves on, items of at least 32 k-blocks.
    plan.dynamic = (plan.items >= 4 * clusters && plan.k_blocks >= 32) ? 1u : 0u;
    if (flags & FK_GEMM_ORDER_STATIC) plan.dynamic = 0;
    if (flags & FK_GEMM_ORDER_FEED) plan.dynamic = plan.items > clusters ? 1u : 0u;
    const uint32_t grid = 2 * (plan.dynamic ? plan.items : plan.items < clusters ? plan.items : clusters);
    if (plan.tile_n == gemm::kBlockN) {
        gemm::gemm_bf16_pair_kernel<false, false><<<grid, gemm::kThreads, gemm::kSharedBytes,
                                                    static_cast<cudaStream_t>(stream)>>>(
            *static_cast<const CUtensorMap*>(a_map), *static_cast<const CUtensorMap*>(b_map),
            *static_cast<const CUtensorMap*>(c_map), *static_cast<const CUtensorMap*>(c_narrow_map), plan, device_status);
    } else {
        const int wide_admitted = fk_admit_shared_plan(
            reinterpret_cast<const void*>(gemm::gemm_bf16_pair_kernel<false, true>), gemm::kSharedBytes, &limit);
        if (wide_admitted != FK_OK) return wide_admitted;
        gemm::gemm_bf16_pair_kernel<false, true><<<grid, gemm::kThreads, gemm::kSharedBytes,
                                                   static_cast<cudaStream_t>(stream)>>>(
            *static_cast<const CUtensorMap*>(a_map), *static_cast<const CUtensorMap*>(b_map),
            *static_cast<const CUtensorMap*>(c_map), *static_cast<const CUtensorMap*>(c_narrow_map), plan, device_status);
    }
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

extern "C" int fk_gemm_launch_fused(const void* a_map, const void* b_map, const void* c_map,
                                    const void* bias, uint32_t m, uint32_t n, uint32_t k, uint32_t group,
                                    uint32_t flags, void* stream, uint32_t* device_status) {
    return launch_fused(a_map, b_map, c_map, c_map, gemm::kBlockN, bias, m, n, k, group, flags, stream, device_status);
}

extern "C" uint32_t fk_gemm_group(uint32_t m, uint32_t n, uint32_t sm_count) {
    // Items in flight: one per cluster, g tile rows by clusters / g tile columns of the traversal. A tile
    // row's panel of A is twice a tile column's panel of B, so the fewest panel bytes per wave are at
    // g = sqrt(clusters / 2): 6 on 148 SMs (measured: 5-7 level, 8 is 1.5 % behind, 16 is 6 %). A
    // matrix narrower than that window (16384 x 2048: 8 tile columns) is covered whole by any g, and
    // short bands did better there (g = 2-4: 1334-1344 TFLOP/s, 6-8: 1313-1322).
    (void)m;
    const uint32_t clusters = sm_count / 2;
    uint32_t best = 1;
    while (2 * (best + 1) * (best + 1) <= clusters) ++best;
    const uint32_t window_columns = best ? clusters / best : clusters;
    if (n / gemm::kBlockN < window_columns) best = best > 2 ? (2 * best) / 3 : best;
    return best ? best : 1u;
}

extern "C" uint32_t fk_gemm_item_columns(uint32_t m, uint32_t n, uint32_t k, uint32_t flags, uint32_t sm_count) {
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN || k % gemm::kBlockK || sm_count < 2)
        return gemm::kBlockN;
    if (takes_narrow(m, n, k, flags, sm_count)) return gemm::kBlockN;
    return gemm::choose_tile_n(m, n, k, sm_count / 2);
}

extern "C" int fk_gemm_launch_tiled(const void* a_map, const void* b_map, const void* c_map, const void* c_tail_map,
                                    uint32_t item_columns, const void* bias, uint32_t m, uint32_t n, uint32_t k,
                                    uint32_t group, uint32_t flags, void* stream, uint32_t* device_status) {
    if (item_columns != gemm::kBlockN && item_columns != gemm::kBlockN - 32 && item_columns != gemm::kBlockN - 64)
        return fk_fail(FK_ERR_SHAPE, "items are 256, 224 or 192 columns wide, not %u", item_columns);
    if (n % item_columns) return fk_fail(FK_ERR_SHAPE, "items of %u columns do not divide the %u columns of C", item_columns, n);
    if (item_columns == gemm::kBlockN - 32 && !c_tail_map)
        return fk_fail(FK_ERR_INVALID, "items of 224 columns store their last 32 through a map of their own, which is null");
    if (item_columns != gemm::kBlockN) {
        DeviceFacts facts;
        const int known = device_facts(&facts);
        if (known != FK_OK) return known;
        if (takes_narrow(m, n, k, flags, static_cast<uint32_t>(facts.sm_count)))
            return fk_fail(FK_ERR_INVALID, "this launch takes the narrow kernel, whose maps are the 256-column ones");
    }
    return launch_fused(a_map, b_map, c_map, c_tail_map ? c_tail_map : c_map, item_columns, bias, m, n, k, group, flags,
                        stream, device_status);
}

extern "C" int fk_gemm_launch(const void* a_map, const void* b_map, const void* c_map, uint32_t m,
                              uint32_t n, uint32_t k, uint32_t group, uint32_t flags, void* stream,
                              uint32_t* device_status) {
    return fk_gemm_launch_fused(a_map, b_map, c_map, nullptr, m, n, k, group, flags, stream, device_status);
}

extern "C" int fk_gemm_bf16_launch(const void* a_map, const void* b_map, const void* c_map,
                                   uint32_t m, uint32_t n, uint32_t k, uint32_t group, void* stream,
                                   uint32_t* device_status) {
    return fk_gemm_launch(a_map, b_map, c_map, m, n, k, group, 0, stream, device_status);
}

// The three maps `gemm::run` builds (examples/src/gemm.rs:506-513), plus the
// store map for C: dims [n, m] with the caller's leading dimension.
// `tile_n` other than 256: B's box is tile_n / 2 rows, and maps[3] is C's store map with a [32, 32]
// box, not swizzled (maps[3] is not written otherwise).
static int gemm_maps(const void* a, const void* b, void* c, uint32_t m, uint32_t n, uint32_t k,
                     uint32_t ldc, CUtensorMap* maps, uint32_t operand_element = FK_BF16,
                     uint32_t tile_n = gemm::kBlockN) {
    fk_layout_t layout;
    const uint64_t a_extents[2] = {k, m}, b_extents[2] = {k, n}, c_extents[2] = {n, m};
    const uint64_t c_strides[2] = {1, ldc};
    int status = fk_layout_packed(&layout, reinterpret_cast<uint64_t>(a), operand_element, 2, a_extents);
    if (status == FK_OK) status = fk_tensor_map(&maps[0], &layout, gemm::kBlockK, gemm::kBlockM, FK_SWIZZLE_128B);
    if (status == FK_OK) status = fk_layout_packed(&layout, reinterpret_cast<uint64_t>(b), operand_element, 2, b_extents);
    if (status == FK_OK) status = fk_tensor_map(&maps[1], &layout, gemm::kBlockK, tile_n / 2, FK_SWIZZLE_128B);
    if (status == FK_OK) status = fk_layout_strided(&layout, reinterpret_cast<uint64_t>(c), FK_BF16, 2, c_extents, c_strides);
    if (status == FK_OK) status = fk_tensor_map(&maps[2], &layout, gemm::kStageColumns, 32, FK_SWIZZLE_128B);
    if (status == FK_OK && tile_n != gemm::kBlockN) status = fk_tensor_map(&maps[3], &layout, 32, 32, FK_SWIZZLE_NONE);
    return status;
}

extern "C" int fk_gemm_fused(const void* a, const void* b, void* c, const void* bias, uint32_t m,
                             uint32_t n, uint32_t k, uint32_t ldc, uint32_t group, uint32_t flags,
                             void* stream, uint32_t* device_status) {
    if (!a || !b || !c) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN ||
        k % gemm::kBlockK)
        return fk_fail(FK_ERR_SHAPE, "%ux%ux%u does not divide the %ux%ux%u tiling", m, n, k,
                       2 * gemm::kBlockM, gemm::kBlockN, gemm::kBlockK);
    if (ldc < n) return fk_fail(FK_ERR_SHAPE, "ldc %u is narrower than the %u columns of C", ldc, n);
    // The maps are this call's own, so the wide kernel's items may be as wide as fills the waves best.
    uint32_t tile_n = gemm::kBlockN;
    DeviceFacts facts;
    if (device_facts(&facts) == FK_OK && facts.sm_count >= 2 &&
        !takes_narrow(m, n, k, flags, static_cast<uint32_t>(facts.sm_count)))
        tile_n = gemm::choose_tile_n(m, n, k, static_cast<uint32_t>(facts.sm_count) / 2);
    alignas(64) CUtensorMap maps[4];
    const int status = gemm_maps(a, b, c, m, n, k, ldc, maps, (flags & FK_GEMM_F16_OPERANDS) ? FK_F16 : FK_BF16, tile_n);
    if (status != FK_OK) return status;
    return launch_fused(&maps[0], &maps[1], &maps[2], tile_n != gemm::kBlockN ? &maps[3] : &maps[2], tile_n, bias, m, n,
                        k, group, flags, stream, device_status);
}

// ---- launches under one wave: K split across the idle clusters, partial sums in a workspace
//
// With fewer items than clusters most SMs idle while a few walk all of K: 1024 x 1024 x 16384 keeps
// 16 clusters busy for 256 k-blocks each. Splitting every item's k-blocks into `splits` runs gives
// every cluster a run; the runs meet in an fp32 workspace (the bf16 reduce-add of
// FK_GEMM_ACCUMULATE would round once per run) and the last to arrive rounds once.
namespace {

// Measured on B200 (back-to-back launches, wide kernel in one launch / split / cuBLAS, microseconds):
// 1024 x 1024 x 4096: 27 / 37 / 12; 1024 x 1024 x 8192: 66 / 39 / 19; 1024 x 1024 x 16384: 91 / 51 / 34;
// 512 x 512 x 16384: 86 / 38 / 23; 256 x 256 x 32768: 162 / 37 / 19. The runs' fp32 tiles cross the L2
// twice (splits x M x N x 4 bytes added, M x N x 4 read back and cleared), and the narrow kernel with K
// cut across a cluster of four beats the split wherever it has tiles enough (512 x 512 x 16384: 26 us,
// 1024 x 1024 x 16384: 38), so what is left for this path is a handful of tiles under a very deep K,
// where four CTAs a tile are still too few: at most 16 narrow tiles, from 512 k-blocks on, in runs of
// at least 32.
constexpr uint32_t kMinSplitDepth = 512;
constexpr uint32_t kMinSplitBlocks = 32;
constexpr uint32_t kMaxSplitTiles = 16;

// How a shape would be split on `clusters` resident clusters: 1 = not at all.
uint32_t split_count(const gemm::Schedule& plan, uint32_t clusters) {
    const uint64_t narrow_tiles = uint64_t(plan.m / gemm::narrow::kTile) * (plan.tiles_n * (gemm::kBlockN / gemm::narrow::kTile));
    if (plan.items == 0 || plan.items * 2 > clusters || plan.k_blocks < kMinSplitDepth || narrow_tiles > kMaxSplitTiles)
        return 1;
    const uint32_t by_clusters = clusters / plan.items;
    const uint32_t by_depth = plan.k_blocks / kMinSplitBlocks;
    const uint32_t splits = by_clusters < by_depth ? by_clusters : by_depth;
    return splits < 2 ? 1 : splits;
}

uint64_t arrivals_bytes(const gemm::Schedule& plan) { return uint64_t(plan.items) * 2 * gemm::kEpilogueWarps * 4; }

}  // namespace

extern "C" uint64_t fk_gemm_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, uint32_t sm_count) {
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN || k % gemm::kBlockK) return 0;
    const uint32_t clusters = sm_count / 2;
    if (clusters == 0) return 0;
    const gemm::Schedule plan = gemm::schedule(m, n, k, 1, clusters);
    if (split_count(plan, clusters) == 1) return 0;
    return uint64_t(m) * n * 4 + arrivals_bytes(plan);
}

extern "C" int fk_gemm_fused_workspace(const void* a, const void* b, void* c, const void* bias, uint32_t m,
                                       uint32_t n, uint32_t k, uint32_t ldc, uint32_t group, uint32_t flags,
                                       void* workspace, uint64_t workspace_bytes, void* stream,
                                       uint32_t* device_status) {
    DeviceFacts facts;
    const int known = device_facts(&facts);
    if (known != FK_OK) return known;
    const uint64_t wanted = fk_gemm_workspace_bytes(m, n, k, static_cast<uint32_t>(facts.sm_count));
    // Shapes that fill a wave, and callers without a workspace, take the one-launch path (which
    // also reports every argument error).
    if (wanted == 0 || !workspace) return fk_gemm_fused(a, b, c, bias, m, n, k, ldc, group, flags, stream, device_status);
    if (workspace_bytes < wanted)
        return fk_fail(FK_ERR_TOO_LARGE, "%ux%ux%u splits K over a workspace of %llu bytes; %llu were given", m, n, k,
                       (unsigned long long)wanted, (unsigned long long)workspace_bytes);
    if (reinterpret_cast<uintptr_t>(workspace) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "the workspace wants 16-byte alignment");
    if (!a || !b || !c) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (ldc < n) return fk_fail(FK_ERR_SHAPE, "ldc %u is narrower than the %u columns of C", ldc, n);
    if (flags & ~(FK_GEMM_F16_OPERANDS | FK_GEMM_ACCUMULATE | FK_GEMM_RELU | FK_GEMM_TILE_WIDE | FK_GEMM_ORDER_STATIC))
        return fk_fail(FK_ERR_INVALID, "unknown GEMM flags 0x%x for a launch that splits K", flags);
    if (reinterpret_cast<uintptr_t>(bias) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "the bias vector wants 16-byte alignment");
    if (group == 0) return fk_fail(FK_ERR_SHAPE, "a traversal group width of 0 has no tiles in it");

    alignas(64) CUtensorMap maps[4];
    int status = gemm_maps(a, b, c, m, n, k, ldc, maps, (flags & FK_GEMM_F16_OPERANDS) ? FK_F16 : FK_BF16);
    if (status != FK_OK) return status;
    fk_layout_t layout;
    const uint64_t extents[2] = {n, m};
    status = fk_layout_packed(&layout, reinterpret_cast<uint64_t>(workspace), FK_F32, 2, extents);
    if (status == FK_OK) status = fk_tensor_map(&maps[3], &layout, 32, 32, FK_SWIZZLE_128B);
    if (status != FK_OK) return status;

    uint32_t limit = 0;
    const int admitted = fk_admit_shared_plan(reinterpret_cast<const void*>(gemm::gemm_bf16_pair_kernel<true, false>),
                                              gemm::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;
    const uint32_t clusters = static_cast<uint32_t>(facts.sm_count) / 2;
    gemm::Schedule plan = gemm::schedule(m, n, k, group, clusters, flags);
    plan.bias = static_cast<const uint16_t*>(bias);
    plan.splits = split_count(plan, clusters);
    plan.split_blocks = (plan.k_blocks + plan.splits - 1) / plan.splits;
    plan.splits = (plan.k_blocks + plan.split_blocks - 1) / plan.split_blocks;  // no empty run
    plan.partial = static_cast<float*>(workspace);
    plan.arrivals = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(workspace) + uint64_t(m) * n * 4);
    const uint32_t units = plan.items * plan.splits;
    const uint32_t grid = 2 * (units < clusters ? units : clusters);
    gemm::gemm_bf16_pair_kernel<true, false><<<grid, gemm::kThreads, gemm::kSharedBytes, static_cast<cudaStream_t>(stream)>>>(
        maps[0], maps[1], maps[2], maps[3], plan, device_status);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

extern "C" int fk_gemm(const void* a, const void* b, void* c, uint32_t m, uint32_t n, uint32_t k,
                       uint32_t ldc, uint32_t group, uint32_t flags, void* stream,
                       uint32_t* device_status) {
    return fk_gemm_fused(a, b, c, nullptr, m, n, k, ldc, group, flags, stream, device_status);
}

extern "C" int fk_gemm_bf16(const void* a, const void* b, void* c, uint32_t m, uint32_t n,
                            uint32_t k, uint32_t ldc, uint32_t group, void* stream,
                            uint32_t* device_status) {
    return fk_gemm(a, b, c, m, n, k, ldc, group, 0, stream, device_status);
}

// Streams and events of the pipelined host-buffer entry, one set per device, created on first use.
namespace {
constexpr uint32_t kHostChunks = 16;
struct HostPipeline {
    cudaStream_t upload = nullptr, compute = nullptr, download = nullptr;
    cudaEvent_t b_ready = nullptr, a_ready[kHostChunks] = {}, c_ready[kHostChunks] = {}, idle = nullptr;
};
std::mutex host_pipeline_guard;
HostPipeline host_pipelines[64];

int host_pipeline(HostPipeline** out) {
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    if (device >= 64) return fk_fail(FK_ERR_INVALID, "device index out of range");
    std::lock_guard<std::mutex> lock(host_pipeline_guard);
    HostPipeline& pipe = host_pipelines[device];
    if (!pipe.upload) {
        FK_CUDA(cudaStreamCreateWithFlags(&pipe.upload, cudaStreamNonBlocking));
        FK_CUDA(cudaStreamCreateWithFlags(&pipe.compute, cudaStreamNonBlocking));
        FK_CUDA(cudaStreamCreateWithFlags(&pipe.download, cudaStreamNonBlocking));
        FK_CUDA(cudaEventCreateWithFlags(&pipe.b_ready, cudaEventDisableTiming));
        FK_CUDA(cudaEventCreateWithFlags(&pipe.idle, cudaEventDisableTiming));
        for (uint32_t i = 0; i < kHostChunks; ++i) {
            FK_CUDA(cudaEventCreateWithFlags(&pipe.a_ready[i], cudaEventDisableTiming));
            FK_CUDA(cudaEventCreateWithFlags(&pipe.c_ready[i], cudaEventDisableTiming));
        }
    }
    *out = &pipe;
    return FK_OK;
}
}  // namespace

static int host_shape_check(const void* a, const void* b, const void* c, uint32_t m, uint32_t n, uint32_t k,
                            uint32_t group) {
    if (!a || !b || !c) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (m == 0 || n == 0 || k == 0 || m % (2 * gemm::kBlockM) || n % gemm::kBlockN || k % gemm::kBlockK)
        return fk_fail(FK_ERR_SHAPE, "%ux%ux%u does not divide the %ux%ux%u tiling", m, n, k,
                       2 * gemm::kBlockM, gemm::kBlockN, gemm::kBlockK);
    if (group == 0) return fk_fail(FK_ERR_SHAPE, "a traversal group width of 0 has no tiles in it");
    return FK_OK;
}

// Upload, compute and read-back overlap: B goes up first, then A in blocks of rows; the GEMM of a
// block starts when its rows of A have landed, and its rows of C go back while later blocks upload and
// compute. Row blocks keep every copy contiguous on both sides. PCIe is full duplex, so the whole call
// costs about the upload alone plus the last block's GEMM and read-back; done in sequence it cost
// upload + compute + read-back. The copies overlap only from page-locked host memory; from pageable
// memory the call is still correct. One call at a time per device: the staging buffers, streams,
// events and status words are the device's, so the call holds the device's guard from its first
// enqueue to its last wait, and a second thread's call on the same device waits its turn.
extern "C" int fk_gemm_bf16_host(const uint16_t* a_host, const uint16_t* b_host, uint16_t* c_host,
                                 uint32_t m, uint32_t n, uint32_t k, uint32_t group) {
    int status = host_shape_check(a_host, b_host, c_host, m, n, k, group);
    if (status != FK_OK) return status;
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> call(device_call_guard(device));
    const size_t a_bytes = size_t(m) * k * 2, b_bytes = size_t(n) * k * 2, c_bytes = size_t(m) * n * 2;
    void *a = nullptr, *b = nullptr, *c = nullptr;
    uint32_t* status_words = nullptr;
    HostPipeline* pipe = nullptr;
    status = scratch(0, a_bytes, &a);
    if (status == FK_OK) status = scratch(1, b_bytes, &b);
    if (status == FK_OK) status = scratch(2, c_bytes, &c);
    if (status == FK_OK) status = scratch_status(&status_words);
    if (status == FK_OK) status = host_pipeline(&pipe);
    if (status != FK_OK) return status;

    // Whole 512-row tiles per block, at most kHostChunks blocks.
    const uint32_t tile_rows = 2 * gemm::kBlockM;
    const uint32_t tiles = m / tile_rows;
    const uint32_t chunk = ((tiles + kHostChunks - 1) / kHostChunks) * tile_rows;
    const uint32_t chunks = (m + chunk - 1) / chunk;

    // Everything is enqueued inside this lambda so that, whatever fails part-way, the three
    // streams are drained below before the call returns: the caller may free or reuse its host
    // buffers the moment it has the return code.
    const auto enqueue = [&]() -> int {
        // The staging buffers are shared with earlier work on the default stream: start after it.
        FK_CUDA(cudaEventRecord(pipe->idle, nullptr));
        FK_CUDA(cudaStreamWaitEvent(pipe->upload, pipe->idle, 0));
        FK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->idle, 0));
        FK_CUDA(cudaStreamWaitEvent(pipe->download, pipe->idle, 0));
        FK_CUDA(cudaMemsetAsync(status_words, 0, 32, pipe->compute));
        FK_CUDA(cudaMemcpyAsync(b, b_host, b_bytes, cudaMemcpyHostToDevice, pipe->upload));
        FK_CUDA(cudaEventRecord(pipe->b_ready, pipe->upload));
        FK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->b_ready, 0));
        for (uint32_t i = 0; i < chunks; ++i) {
            const uint32_t row0 = i * chunk, rows = (m - row0 < chunk) ? m - row0 : chunk;
            uint8_t* a_chunk = static_cast<uint8_t*>(a) + size_t(row0) * k * 2;
            uint8_t* c_chunk = static_cast<uint8_t*>(c) + size_t(row0) * n * 2;
            FK_CUDA(cudaMemcpyAsync(a_chunk, a_host + size_t(row0) * k, size_t(rows) * k * 2,
                                    cudaMemcpyHostToDevice, pipe->upload));
            FK_CUDA(cudaEventRecord(pipe->a_ready[i], pipe->upload));
            FK_CUDA(cudaStreamWaitEvent(pipe->compute, pipe->a_ready[i], 0));
            const int launched = fk_gemm_bf16(a_chunk, b, c_chunk, rows, n, k, n, group, pipe->compute, status_words);
            if (launched != FK_OK) return launched;
            FK_CUDA(cudaEventRecord(pipe->c_ready[i], pipe->compute));
            FK_CUDA(cudaStreamWaitEvent(pipe->download, pipe->c_ready[i], 0));
            FK_CUDA(cudaMemcpyAsync(c_host + size_t(row0) * n, c_chunk, size_t(rows) * n * 2,
                                    cudaMemcpyDeviceToHost, pipe->download));
        }
        return FK_OK;
    };
    status = enqueue();
    // Whatever happened, leave no work of this call in flight behind the return. Each wait carries
    // the launch deadline (src/watchdog.rs:300-332): a wedged device yields FK_ERR_TIMEOUT, not a hang.
    const int up = wait_stream(pipe->upload);
    const int run = wait_stream(pipe->compute);
    const int down = wait_stream(pipe->download);
    if (status != FK_OK) return status;
    if (up != FK_OK) return up;
    if (run != FK_OK) return run;
    if (down != FK_OK) return down;
    return fk_status_check(status_words, pipe->compute);
}

// ------------------------------------------------------------------ no-allocation variant
//
// fk_gemm_bf16_host stages its operands in device buffers it gets from cudaMalloc. Some callers
// must never reach the CUDA allocator from this call: a serving loop whose latency budget cannot
// absorb the device-wide synchronisation cudaMalloc and cudaFree imply, or a process whose device
// memory is already handed out in full to another pool, where a late cudaMalloc may simply fail.
// For them the same staging (A, B, C and the status words) lives in one array that is part of
// the library image, of a fixed, modest size.

namespace {

constexpr size_t kStaticOperandBytes = 8u << 20;  // each of A, B and C: at most 8 MiB
constexpr size_t kStaticStatusBytes = 256;
// Held by every GPU that loads the library, until the process exits.
static __device__ __align__(256) uint8_t fk_static_scratch[3 * kStaticOperandBytes + kStaticStatusBytes];

// The array's name is only a host-side handle; the device address is looked up once per device.
int static_scratch(uint8_t** out) {
    static std::mutex guard;
    static uint8_t* base[64] = {};
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fk_fail(FK_ERR_INVALID, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(guard);
    if (!base[device]) {
        void* address = nullptr;
        FK_CUDA(cudaGetSymbolAddress(&address, fk_static_scratch));
        base[device] = static_cast<uint8_t*>(address);
    }
    *out = base[device];
    return FK_OK;
}

}  // namespace

extern "C" int fk_gemm_bf16_host_noalloc(const uint16_t* a_host, const uint16_t* b_host,
                                         uint16_t* c_host, uint32_t m, uint32_t n, uint32_t k,
                                         uint32_t group) {
    // Every refusal comes before the first enqueue: a refused call has touched nothing.
    int status = host_shape_check(a_host, b_host, c_host, m, n, k, group);
    if (status != FK_OK) return status;
    const size_t a_bytes = size_t(m) * k * 2, b_bytes = size_t(n) * k * 2, c_bytes = size_t(m) * n * 2;
    if (a_bytes > kStaticOperandBytes || b_bytes > kStaticOperandBytes || c_bytes > kStaticOperandBytes)
        return fk_fail(FK_ERR_TOO_LARGE,
                       "%ux%ux%u needs %zu / %zu / %zu bytes for A / B / C; the built-in staging holds "
                       "%zu bytes each (use fk_gemm_bf16_host for larger shapes)",
                       m, n, k, a_bytes, b_bytes, c_bytes, kStaticOperandBytes);
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> call(device_call_guard(device));
    uint8_t* scratch_base = nullptr;
    status = static_scratch(&scratch_base);
    if (status != FK_OK) return status;
    void* a = scratch_base;
    void* b = scratch_base + kStaticOperandBytes;
    void* c = scratch_base + 2 * kStaticOperandBytes;
    uint32_t* status_words = reinterpret_cast<uint32_t*>(scratch_base + 3 * kStaticOperandBytes);
    cudaStream_t stream = nullptr;
    const auto enqueue = [&]() -> int {
        // The array keeps the previous call's contents: the status words must start at zero. A, B
        // and C are overwritten in full by this call before anything reads them.
        FK_CUDA(cudaMemsetAsync(status_words, 0, 32, stream));
        FK_CUDA(cudaMemcpyAsync(a, a_host, a_bytes, cudaMemcpyHostToDevice, stream));
        FK_CUDA(cudaMemcpyAsync(b, b_host, b_bytes, cudaMemcpyHostToDevice, stream));
        const int launched = fk_gemm_bf16(a, b, c, m, n, k, n, group, stream, status_words);
        if (launched != FK_OK) return launched;
        FK_CUDA(cudaMemcpyAsync(c_host, c, c_bytes, cudaMemcpyDeviceToHost, stream));
        return FK_OK;
    };
    status = enqueue();
    if (status != FK_OK) {
        wait_stream(stream);  // no copy of this call may still be reading the caller's buffers
        return status;
    }
    return fk_status_check(status_words, stream);
}
