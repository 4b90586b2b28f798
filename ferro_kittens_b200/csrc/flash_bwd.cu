// Flash-attention backward, D = 128, for sm_100a: dQ, dK, dV from Q, K, V, O, dO and the forward's
// log-sum-exp, bf16 in and out, fp32 accumulation.
//
// The reference has no backward kernel; it carries the pieces one is built from -- the
// transposed-operand MMAs (`mma_atb`, `mma_atbt`, src/mma.rs:314-376), the transposed causal mask
// (`make_causal_t_at`, src/reg.rs:1432-1434) and the row/column vector loads for a saved LSE
// (src/global.rs:573-654) -- and its forward's output is this kernel's input. The arithmetic is the
// standard one:
//
//   P = exp(scale S - lse),  S = Q K^T          dV = P^T dO
//   dP = dO V^T,  delta = rowsum(dO * O)         dS = scale P * (dP - delta)
//   dQ = dS K                                    dK = dS^T Q
//
// Three launches, nothing atomic, results independent of scheduling:
//   1. `stats`: -delta and -lse * log2(e) per query row (memory-bound, reads O and dO once).
//   2. one CTA per 128-key block owns K_j, V_j and the accumulators dV_j, dK_j in tensor memory and
//      streams the query blocks past them. It computes the TRANSPOSED tiles S^T = K_j Q_i^T and
//      dP^T = V_j dO_i^T so that keys are the tensor-memory lanes: P^T and dS^T are then A operands
//      from tensor memory of dV_j += P^T dO_i and dK_j += dS^T Q_i, with dO_i and Q_i read MN-major
//      from the same shared tiles the first two MMAs read K-major.
//   3. one CTA per 128-query block owns Q_i, dO_i and dQ_i and streams the key blocks: S = Q_i K_j^T,
//      dP = dO_i V_j^T, dQ_i += dS K_j. (S and dP are computed twice overall: 7 tile MMAs per tile
//      pair instead of 5, the price of not adding into dQ from many CTAs.)
// Launches 2 and 3 are one kernel template. The element-wise step is split in two (P from S, then dS
// from dP and the P kept in registers) and the MMA issue order interleaves blocks, so that the tensor
// pipe works on one of the two fp32 tiles while the element-wise warps work on the other. Roles per
// CTA: warps 0-7 the element-wise step (two warps per lane quadrant, 64 columns each; no reduction
// crosses a thread; four per quadrant measured slower), warp 8 the loader (TMA tiles through a
// three-slot ring for the tile a block reads last, the per-column statistics by bulk copy), warp 9 the
// MMA issue, warp 10 a second loader (a two-slot ring for the other streamed tile). Tensor memory: T1 (S or S^T; bf16 P over it) |
// T2 (dP; bf16 dS over it) |
// accumulator 0 | accumulator 1, 128 columns each. Every wait is bounded.

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
namespace flash_bwd {

constexpr uint32_t kRows = 128;  // rows of every tile: a query block or a key block
constexpr uint32_t kHead = 128;
// The two streamed tiles of a block leave their slots at different times (the second MMA pair
// reads x0 last, after dS is ready), so each has its own ring; a single two-slot ring made every
// block wait out a TMA round trip.
constexpr uint32_t kSlots0 = 3;  // Q_i (key-block owners) / K_j: read by the first and the last product of a block
constexpr uint32_t kSlots1 = 2;  // dO_i / V_j
constexpr uint32_t kSlotsStats = 2;
constexpr uint32_t kElementWarps = 8;     // two per lane quadrant, 64 columns of T each (four measured slower)
constexpr uint32_t kThreadColumns = 64;   // columns of T a thread owns
constexpr uint32_t kLoaderWarp = kElementWarps;       // x0 ring and the column statistics
constexpr uint32_t kMmaWarp = kElementWarps + 1;
constexpr uint32_t kLoaderWarp1 = kElementWarps + 2;  // x1 ring
constexpr uint32_t kThreads = (kElementWarps + 3) * 32;
constexpr uint32_t kSubtileBytes = kRows * 64 * 2;
constexpr uint32_t kTileBytes = 2 * kSubtileBytes;
constexpr uint32_t kStatsBytes = 2 * kRows * 4;  // lse * log2(e) and delta of one query block
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kT1 = 0, kT2 = 128, kAcc0 = 256, kAcc1 = 384;

struct Plan {
    SharedPlan resident, ring0, ring1, stats, resident_full, full0, empty0, full1, empty1, stats_full, stats_empty,
        t1_full, t2_full, p_ready, ds_ready, acc_done, tmem_slot, stop, end;
    constexpr Plan()
        : resident(SharedPlan{}.tile_ring(kRows, kHead, 2, 2)),
          ring0(resident.tile_ring(kRows, kHead, 2, kSlots0)),
          ring1(ring0.tile_ring(kRows, kHead, 2, kSlots1)),
          stats(ring1.reserve(kSlotsStats * kStatsBytes, 16)),
          resident_full(stats.semaphore()),
          full0(resident_full.semaphores(kSlots0)),
          empty0(full0.semaphores(kSlots0)),
          full1(empty0.semaphores(kSlots1)),
          empty1(full1.semaphores(kSlots1)),
          stats_full(empty1.semaphores(kSlotsStats)),
          stats_empty(stats_full.semaphores(kSlotsStats)),
          t1_full(stats_empty.semaphore()),
          t2_full(t1_full.semaphore()),
          p_ready(t2_full.semaphore()),
          ds_ready(p_ready.semaphore()),
          acc_done(ds_ready.semaphore()),
          tmem_slot(acc_done.tmem_slot()),
          stop(tmem_slot.word()),
          end(stop) {}
};
constexpr Plan kPlan{};
constexpr uint32_t kBaseAlign = 1024;
constexpr uint32_t kSharedBytes = static_cast<uint32_t>(kPlan.end.bytes());
static_assert(kSharedBytes <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");

enum StallCode : uint32_t {
    kStallLoader = 0x401,
    kStallMmaResident = 0x402,
    kStallMmaStream = 0x403,
    kStallMmaP = 0x404,
    kStallElementT = 0x405,
    kStallElementAcc = 0x406,
    kStallMmaDs = 0x407,
    kStallElementT2 = 0x408,
    kMisaligned = 0x4ff,
};

// Of the 16 score pairs of a 32-column chunk, those whose bit is set take 2^x from a polynomial on
// the FMA pipe instead of the ex2 unit (the forward's trick, same polynomial). Half of them is the
// measured optimum here: 870 vs 773 TFLOP/s non-causal, 853 vs 806 causal in back-to-back launches;
// three quarters and more are slower than none.
constexpr uint32_t kPolyMask = 0x5555u;

// -lse * log2(e) and -delta = -rowsum(dO * O) (negated: they enter as addends), one query row per 16 lanes.
__global__ void __launch_bounds__(256) stats_kernel(const uint16_t* __restrict__ o, const uint16_t* __restrict__ d_o,
                                                    const float* __restrict__ lse, float* __restrict__ stats,
                                                    uint32_t planes, uint32_t seq) {
    const uint64_t rows = static_cast<uint64_t>(planes) * seq;
    const uint32_t lane = threadIdx.x & 31, sub = lane >> 4, chunk = lane & 15;
    const uint64_t warps = static_cast<uint64_t>(gridDim.x) * (blockDim.x >> 5);
    for (uint64_t pair = static_cast<uint64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); 2 * pair < rows;
         pair += warps) {
        const uint64_t row = 2 * pair + sub;
        float total = 0.0f;
        if (row < rows) {
            const uint4 a = *reinterpret_cast<const uint4*>(o + row * kHead + 8 * chunk);
            const uint4 b = *reinterpret_cast<const uint4*>(d_o + row * kHead + 8 * chunk);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i)
                total += __uint_as_float(aw[i] << 16) * __uint_as_float(bw[i] << 16) +
                         __uint_as_float(aw[i] & 0xffff0000u) * __uint_as_float(bw[i] & 0xffff0000u);
        }
#pragma unroll
        for (uint32_t mask = 8; mask > 0; mask >>= 1) total += __shfl_xor_sync(0xffffffffu, total, mask);
        if (row < rows && chunk == 0) {
            const uint64_t plane = row / seq, at = row % seq;
            stats[(2 * plane) * seq + at] = -lse[row] * 1.4426950408889634f;
            stats[(2 * plane + 1) * seq + at] = -total;
        }
    }
}

// KV = true: the CTA owns a key block (resident K_j, V_j; streams Q_i, dO_i; lanes are keys).
// KV = false: it owns a query block (resident Q_i, dO_i; streams K_j, V_j; lanes are queries).
template <bool KV>
__global__ void __launch_bounds__(kThreads, 1)
    backward_kernel(const __grid_constant__ CUtensorMap r0_map, const __grid_constant__ CUtensorMap r1_map,
                    const __grid_constant__ CUtensorMap x0_map, const __grid_constant__ CUtensorMap x1_map,
                    const __grid_constant__ CUtensorMap out0_map, const __grid_constant__ CUtensorMap out1_map,
                    const float* __restrict__ stats, uint32_t seq, float scale, uint32_t causal, uint32_t* status) {
    extern __shared__ __align__(1024) uint8_t dynamic_shared[];
    const uint32_t base = smem_u32(dynamic_shared);
    if (base & (kBaseAlign - 1)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0u, static_cast<uint32_t>(kMisaligned));
        return;
    }
    const uint32_t resident = base + kPlan.resident.at;
    const uint32_t ring0 = base + kPlan.ring0.at;
    const uint32_t ring1 = base + kPlan.ring1.at;
    const uint32_t stats_smem = base + kPlan.stats.at;
    const uint32_t resident_full = base + kPlan.resident_full.at;
    const uint32_t full0 = base + kPlan.full0.at, empty0 = base + kPlan.empty0.at;
    const uint32_t full1 = base + kPlan.full1.at, empty1 = base + kPlan.empty1.at;
    const uint32_t stats_full = base + kPlan.stats_full.at, stats_empty = base + kPlan.stats_empty.at;
    const uint32_t t1_full = base + kPlan.t1_full.at;
    const uint32_t t2_full = base + kPlan.t2_full.at;
    const uint32_t p_ready = base + kPlan.p_ready.at;
    const uint32_t ds_ready = base + kPlan.ds_ready.at;
    const uint32_t acc_done = base + kPlan.acc_done.at;
    const uint32_t slot = base + kPlan.tmem_slot.at;
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.stop.at);
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.tmem_slot.at);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t owner = blockIdx.x;  // the key block (KV) or query block this CTA owns
    const uint32_t plane = blockIdx.y;
    const uint32_t blocks = seq / kRows;
    // Streamed blocks: all of them, or under a causal mask the query blocks at and after the key
    // block (KV) / the key blocks up to and including the query block.
    const uint32_t first = (causal && KV) ? owner : 0u;
    const uint32_t count = causal ? (KV ? blocks - owner : owner + 1u) : blocks;

    if (threadIdx.x == 0) {
        mbar_init(resident_full, 1);
        for (uint32_t i = 0; i < kSlots0; ++i) {
            mbar_init(full0 + 8 * i, 1);
            mbar_init(empty0 + 8 * i, 1);
        }
        for (uint32_t i = 0; i < kSlots1; ++i) {
            mbar_init(full1 + 8 * i, 1);
            mbar_init(empty1 + 8 * i, 1);
        }
        for (uint32_t i = 0; i < kSlotsStats; ++i) {
            mbar_init(stats_full + 8 * i, 1);
            mbar_init(stats_empty + 8 * i, kElementWarps);
        }
        mbar_init(t1_full, 1);
        mbar_init(t2_full, 1);
        mbar_init(p_ready, kElementWarps);
        mbar_init(ds_ready, kElementWarps);
        mbar_init(acc_done, 1);
        *stop_flag = 0;
        fence_mbarrier_init();
        prefetch_tensormap(&r0_map);
        prefetch_tensormap(&r1_map);
        prefetch_tensormap(&x0_map);
        prefetch_tensormap(&x1_map);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<1>(slot, kTmemColumns);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot_ptr;
    // The waits suspend in try_wait: polling measured no better here (it pays in the forward).
    const StallSite site{status, stop_flag, 0, kWaitBudgetCycles, false};

    if (warp == kLoaderWarp) {
        // ------------------------------------------------ loader: resident tiles, the x0 ring, the statistics
        if (lane == 0) {
            mbar_arrive_expect_tx(resident_full, 2 * kTileBytes);
            for (uint32_t half = 0; half < 2; ++half) {
                tma_load_3d(resident + half * kSubtileBytes, &r0_map, static_cast<int>(64 * half),
                            static_cast<int>(kRows * owner), static_cast<int>(plane), resident_full);
                tma_load_3d(resident + kTileBytes + half * kSubtileBytes, &r1_map, static_cast<int>(64 * half),
                            static_cast<int>(kRows * owner), static_cast<int>(plane), resident_full);
            }
            for (uint32_t n = 0; n < count; ++n) {
                const uint32_t s = n % kSlots0, block = first + n;
                if (!mbar_wait(empty0 + 8 * s, ((n / kSlots0) & 1u) ^ 1u, site, kStallLoader, n)) break;
                mbar_arrive_expect_tx(full0 + 8 * s, kTileBytes);
                for (uint32_t half = 0; half < 2; ++half)
                    tma_load_3d(ring0 + s * kTileBytes + half * kSubtileBytes, &x0_map, static_cast<int>(64 * half),
                                static_cast<int>(kRows * block), static_cast<int>(plane), full0 + 8 * s);
                if (KV) {
                    // The streamed query block's statistics, one value per COLUMN of the transposed tiles.
                    const uint32_t ss = n % kSlotsStats;
                    if (!mbar_wait(stats_empty + 8 * ss, ((n / kSlotsStats) & 1u) ^ 1u, site, kStallLoader, n)) break;
                    mbar_arrive_expect_tx(stats_full + 8 * ss, kStatsBytes);
                    const float* source = stats + (2 * static_cast<size_t>(plane)) * seq + kRows * block;
                    for (uint32_t which = 0; which < 2; ++which)
                        asm volatile(
                            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                stats_smem + ss * kStatsBytes + which * kRows * 4),
                            "l"(source + which * static_cast<size_t>(seq)), "r"(kRows * 4), "r"(stats_full + 8 * ss)
                            : "memory");
                }
            }
        }
    } else if (warp == kLoaderWarp1) {
        // ------------------------------------------------ loader: the x1 ring
        if (lane == 0) {
            for (uint32_t n = 0; n < count; ++n) {
                const uint32_t s = n % kSlots1, block = first + n;
                if (!mbar_wait(empty1 + 8 * s, ((n / kSlots1) & 1u) ^ 1u, site, kStallLoader, n)) break;
                mbar_arrive_expect_tx(full1 + 8 * s, kTileBytes);
                for (uint32_t half = 0; half < 2; ++half)
                    tma_load_3d(ring1 + s * kTileBytes + half * kSubtileBytes, &x1_map, static_cast<int>(64 * half),
                                static_cast<int>(kRows * block), static_cast<int>(plane), full1 + 8 * s);
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------ MMA issue
        // One elected thread runs the whole role, waits, MMAs and commits: the compiler then knows the
        // region is single-threaded and emits the tight issue sequence (see the note at elect_one).
        constexpr uint32_t idesc_ss = instruction_descriptor(kRows, kRows, false, false);
        constexpr uint32_t idesc_ts = instruction_descriptor(kRows, kHead, false, true);
        if (elect_one()) {
        auto wait = [&](uint32_t bar, uint32_t parity, uint32_t code, uint32_t detail) {
            const bool ok = mbar_wait(bar, parity, site, code, detail);
            if (ok) tc_fence_after_sync();
            return ok;
        };
        // T = A . B^T over d = 128, both tiles K-major: two stacked [128, 64] subtiles, four K=16 chunks each.
        auto transposed_product = [&](uint32_t t_column, uint32_t a_tile, uint32_t b_tile) {
            const uint64_t a_desc = operand_descriptor(a_tile, kKMajorLeadingBytes);
            const uint64_t b_desc = operand_descriptor(b_tile, kKMajorLeadingBytes);
#pragma unroll
            for (uint32_t chunk = 0; chunk < kHead / 16; ++chunk) {
                const uint64_t step = ((chunk / 4) * kSubtileBytes + (chunk % 4) * kKMajorChunkBytes) >> 4;
                mma_ss<1>(tmem + t_column, a_desc + step, b_desc + step, idesc_ss, chunk != 0);
            }
        };
        // ACC (+)= A . B over the tile's 128 rows: A is the bf16 the element-wise warps left over T
        // (a thread's kThreadColumns contraction rows packed into the first half of its own columns), B the streamed
        // tile read MN-major: 16 rows per chunk, the second 64 head columns one subtile on.
        auto accumulate = [&](uint32_t acc_column, uint32_t t_column, uint32_t b_tile, bool keep) {
            const uint64_t b_desc = operand_descriptor(b_tile, kSubtileBytes);
#pragma unroll
            for (uint32_t chunk = 0; chunk < kRows / 16; ++chunk)
                mma_ts(tmem + acc_column,
                          tmem + t_column + kThreadColumns * (16 * chunk / kThreadColumns) + (16 * chunk % kThreadColumns) / 2,
                          b_desc + ((chunk * kMnMajorChunkBytes) >> 4), idesc_ts, (keep || chunk != 0) ? 1u : 0u);
        };

        // Issue order per block n: [P(n) ready] dV += P^T dO; S(n+1); [dS(n) ready] dK/dQ += dS^T Q;
        // dP(n+1). The tensor pipe runs in issue order, so S(n+1) cannot overwrite P(n) before the MMA
        // that reads it, nor dP(n+1) dS(n); and while the element-wise warps work on one of the two
        // tiles the pipe has the other's products to run. x1(n) is last read by dV's product (key-block
        // owners) or by dP's (query-block owners); x0(n) by the block's last product.
        const auto x0_of = [&](uint32_t n) { return ring0 + (n % kSlots0) * kTileBytes; };
        const auto x1_of = [&](uint32_t n) { return ring1 + (n % kSlots1) * kTileBytes; };
        bool live = wait(resident_full, 0, kStallMmaResident, 0);
        if (live && count != 0) live = wait(full0, 0, kStallMmaStream, 0);
        if (live && count != 0) {
            transposed_product(kT1, resident, x0_of(0));  // S^T = K Q^T   |  S = Q K^T
            mma_commit<1>(t1_full);
            live = wait(full1, 0, kStallMmaStream, 0);
        }
        if (live && count != 0) {
            transposed_product(kT2, resident + kTileBytes, x1_of(0));  // dP^T = V dO^T | dP = dO V^T
            mma_commit<1>(t2_full);
            if (!KV) mma_commit<1>(empty1);
        }
        for (uint32_t n = 0; live && n < count; ++n) {
            const bool more = n + 1 < count;
            if (!wait(p_ready, n & 1u, kStallMmaP, n)) break;
            if (KV) {
                accumulate(kAcc0, kT1, x1_of(n), n != 0);  // dV += P^T dO
                mma_commit<1>(empty1 + 8 * (n % kSlots1));
            }
            if (more) {
                if (!wait(full0 + 8 * ((n + 1) % kSlots0), ((n + 1) / kSlots0) & 1u, kStallMmaStream, n + 1)) break;
                transposed_product(kT1, resident, x0_of(n + 1));
                mma_commit<1>(t1_full);
            }
            if (!wait(ds_ready, n & 1u, kStallMmaDs, n)) break;
            accumulate(kAcc1, kT2, x0_of(n), n != 0);  // dK += dS^T Q  |  dQ += dS K
            mma_commit<1>(empty0 + 8 * (n % kSlots0));
            if (more) {
                if (!wait(full1 + 8 * ((n + 1) % kSlots1), ((n + 1) / kSlots1) & 1u, kStallMmaStream, n + 1)) break;
                transposed_product(kT2, resident + kTileBytes, x1_of(n + 1));
                mma_commit<1>(t2_full);
                if (!KV) mma_commit<1>(empty1 + 8 * ((n + 1) % kSlots1));
            }
        }
        mma_commit<1>(acc_done);
        }
        __syncwarp();
    } else if (warp < kElementWarps) {
        // ------------------------------------------------ element-wise step and epilogue
        const uint32_t part = warp >> 2;            // which kThreadColumns columns of T / head columns of an accumulator
        const uint32_t quadrant = warp & 3u;        // tensor-memory lanes this warp may touch
        const uint32_t row = 32 * quadrant + lane;  // lane of the tiles = row of the owned block
        const uint32_t lane_base = (32 * quadrant) << 16;
        const uint32_t column0 = kThreadColumns * part;
        constexpr uint32_t kChunks = kThreadColumns / 32;
        const float scale_log2 = scale * 1.4426950408889634f;
        const float2 scale_log2_pair = make_float2(scale_log2, scale_log2);
        const float2 scale_pair = make_float2(scale, scale);
        float row_lse = 0.0f, row_delta = 0.0f;  // negated, as the workspace holds them
        if (!KV) {
            row_lse = stats[(2 * static_cast<size_t>(plane)) * seq + kRows * owner + row];
            row_delta = stats[(2 * static_cast<size_t>(plane) + 1) * seq + kRows * owner + row];
        }
        bool live = true;
        for (uint32_t n = 0; live && n < count; ++n) {
            const uint32_t s = n % kSlotsStats, block = first + n;
            // ---- first half of the step: P from S, while the pipe computes dP
            if (!mbar_wait(t1_full, n & 1u, site, kStallElementT, n)) {
                live = false;
                break;
            }
            tc_fence_after_sync();
            if (KV && !mbar_wait(stats_full + 8 * s, (n / kSlotsStats) & 1u, site, kStallElementT, n)) {
                live = false;
                break;
            }
            const bool diagonal = causal && block == owner;
            const uint32_t column_stats = stats_smem + s * kStatsBytes + column0 * 4;
            float2 p[kThreadColumns / 2];
#pragma unroll
            for (uint32_t c = 0; c < kChunks; ++c) {
                uint32_t score[32];
                tmem_ld_32x32(tmem + lane_base + kT1 + column0 + 32 * c, score);
                float2 offset[16];
                if (KV) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        uint32_t words[4];
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3])
                                     : "r"(column_stats + 128 * c + 16 * i));
                        offset[2 * i] = make_float2(__uint_as_float(words[0]), __uint_as_float(words[1]));
                        offset[2 * i + 1] = make_float2(__uint_as_float(words[2]), __uint_as_float(words[3]));
                    }
                }
                tmem_wait_ld();
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) {
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(score[2 * i]), __uint_as_float(score[2 * i + 1])),
                                                scale_log2_pair, KV ? offset[i] : make_float2(row_lse, row_lse));
                    p[16 * c + i] = ((kPolyMask >> i) & 1u) ? exp2_pair_fma(x) : make_float2(ex2_approx(x.x), ex2_approx(x.y));
                }
                if (diagonal) {
                    // KV: lane = key, column = query, visible iff key <= query. Otherwise lane = query.
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const uint32_t column = column0 + 32 * c + 2 * i;
                        if (KV ? column < row : column > row) p[16 * c + i].x = 0.0f;
                        if (KV ? column + 1 < row : column + 1 > row) p[16 * c + i].y = 0.0f;
                    }
                }
                if (KV) {
                    uint32_t p_words[16];
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) p_words[i] = pack_bf16x2(p[16 * c + i].x, p[16 * c + i].y);
                    // Over the first half of this thread's own columns, all of which it has read by now
                    // or (chunk 1's scores) lie in the second half.
                    tmem_st_32x16(tmem + lane_base + kT1 + column0 + 16 * c, p_words);
                }
            }
            if (KV) tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);  // P is in place (KV), and S has been consumed

            // ---- second half: dS from dP and the P still in registers, while the pipe runs dV and S(n+1)
            if (!mbar_wait(t2_full, n & 1u, site, kStallElementT2, n)) {
                live = false;
                break;
            }
            tc_fence_after_sync();
#pragma unroll
            for (uint32_t c = 0; c < kChunks; ++c) {
                uint32_t slope[32];
                tmem_ld_32x32(tmem + lane_base + kT2 + column0 + 32 * c, slope);
                float2 offset[16];
                if (KV) {
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i) {
                        uint32_t words[4];
                        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(words[0]), "=r"(words[1]), "=r"(words[2]), "=r"(words[3])
                                     : "r"(column_stats + kRows * 4 + 128 * c + 16 * i));
                        offset[2 * i] = make_float2(__uint_as_float(words[0]), __uint_as_float(words[1]));
                        offset[2 * i + 1] = make_float2(__uint_as_float(words[2]), __uint_as_float(words[3]));
                    }
                }
                tmem_wait_ld();
                uint32_t ds_words[16];
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) {
                    // dS = scale * P * (dP - delta)
                    const float2 centred = __fadd2_rn(make_float2(__uint_as_float(slope[2 * i]), __uint_as_float(slope[2 * i + 1])),
                                                      KV ? offset[i] : make_float2(row_delta, row_delta));
                    const float2 ds = __fmul2_rn(__fmul2_rn(p[16 * c + i], scale_pair), centred);
                    ds_words[i] = pack_bf16x2(ds.x, ds.y);
                }
                tmem_st_32x16(tmem + lane_base + kT2 + column0 + 16 * c, ds_words);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(ds_ready);
                if (KV) mbar_arrive(stats_empty + 8 * s);  // the block's statistics have been read
            }
        }

        if (live && !mbar_wait(acc_done, 0, site, kStallElementAcc, count)) live = false;
        if (live) {
            tc_fence_after_sync();
            // The resident tiles are dead once the last MMA retired: they stage the two outputs. This
            // warp owns rows [32 q, 32 q + 32) x 64 head columns of an accumulator: one [32, 64] store box.
#pragma unroll 1
            for (uint32_t which = KV ? 0u : 1u; which < 2 && live; ++which) {
                const uint32_t half = column0 / 64;
                const uint32_t subtile = resident + which * kTileBytes + half * kSubtileBytes;
#pragma unroll 1
                for (uint32_t c = 0; c < kChunks; ++c) {
                    uint32_t value[32];
                    tmem_ld_32x32(tmem + lane_base + (which ? kAcc1 : kAcc0) + column0 + 32 * c, value);
                    tmem_wait_ld();
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t* v = value + 8 * i;
                        st_shared_v4(subtile + swizzled_chunk_offset(row, ((column0 + 32 * c) % 64) / 8 + i, 0),
                                     pack_bf16x2(__uint_as_float(v[0]), __uint_as_float(v[1])),
                                     pack_bf16x2(__uint_as_float(v[2]), __uint_as_float(v[3])),
                                     pack_bf16x2(__uint_as_float(v[4]), __uint_as_float(v[5])),
                                     pack_bf16x2(__uint_as_float(v[6]), __uint_as_float(v[7])));
                    }
                }
                fence_proxy_async_shared();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(which ? &out1_map : &out0_map, subtile + 32 * quadrant * 128,
                                 static_cast<int>(64 * half), static_cast<int>(kRows * owner + 32 * quadrant),
                                 static_cast<int>(plane));
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_before_exit();
    }

    // ---------------------------------------------------- teardown
    if (*stop_flag) {
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc<1>(tmem, kTmemColumns);
}

}  // namespace flash_bwd
}  // namespace fk

// ------------------------------------------------------------------ C ABI

using namespace fk;

extern "C" uint32_t fk_flash_bwd_shared_bytes(void) { return flash_bwd::kSharedBytes; }
extern "C" uint32_t fk_flash_bwd_threads(void) { return flash_bwd::kThreads; }
extern "C" uint64_t fk_flash_bwd_workspace_bytes(uint32_t planes, uint32_t seq) {
    return 2ull * planes * seq * sizeof(float);
}

extern "C" int fk_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, void* dq, void* dk, void* dv, float* workspace, uint32_t planes,
                            uint32_t seq, float scale, int causal, void* stream, uint32_t* device_status) {
    if (!q || !k || !v || !o || !d_o || !lse || !dq || !dk || !dv || !workspace)
        return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (seq == 0 || seq % flash_bwd::kRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE, "%u queries x %u heads does not divide the %u queries a tile owns", seq, planes,
                       flash_bwd::kRows);
    if (planes > 65535) return fk_fail(FK_ERR_SHAPE, "%u planes is past the 65535 a launch takes", planes);
    if ((reinterpret_cast<uintptr_t>(workspace) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(d_o)) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "the workspace, O and dO want 16-byte alignment");
    alignas(64) CUtensorMap maps[7];
    const void* loads[4] = {q, k, v, d_o};
    void* stores[3] = {dq, dk, dv};
    int status = FK_OK;
    for (int i = 0; i < 4 && status == FK_OK; ++i)
        status = fk_encode_bf16_panels(&maps[i], reinterpret_cast<uint64_t>(loads[i]), flash_bwd::kRows,
                                       flash_bwd::kHead, seq, planes);
    for (int i = 0; i < 3 && status == FK_OK; ++i)
        status = fk_encode_bf16_panels(&maps[4 + i], reinterpret_cast<uint64_t>(stores[i]), 32, flash_bwd::kHead,
                                       seq, planes);
    if (status != FK_OK) return status;
    uint32_t limit = 0;
    status = fk_admit_shared_plan(reinterpret_cast<const void*>(flash_bwd::backward_kernel<true>),
                                  flash_bwd::kSharedBytes, &limit);
    if (status == FK_OK)
        status = fk_admit_shared_plan(reinterpret_cast<const void*>(flash_bwd::backward_kernel<false>),
                                      flash_bwd::kSharedBytes, &limit);
    if (status != FK_OK) return status;

    cudaStream_t on = static_cast<cudaStream_t>(stream);
    const uint64_t rows = static_cast<uint64_t>(planes) * seq;
    const uint32_t stat_blocks = static_cast<uint32_t>((rows / 2 + 7) / 8 < 148 * 8 ? (rows / 2 + 7) / 8 : 148 * 8);
    flash_bwd::stats_kernel<<<stat_blocks ? stat_blocks : 1, 256, 0, on>>>(
        static_cast<const uint16_t*>(o), static_cast<const uint16_t*>(d_o), lse, workspace, planes, seq);
    FK_CUDA(cudaGetLastError());
    const dim3 grid(seq / flash_bwd::kRows, planes, 1);
    const CUtensorMap &q_map = maps[0], &k_map = maps[1], &v_map = maps[2], &do_map = maps[3];
    const CUtensorMap &dq_map = maps[4], &dk_map = maps[5], &dv_map = maps[6];
    // Key-block owners: resident K, V; streamed Q, dO; outputs dV (accumulator 0) and dK (accumulator 1).
    flash_bwd::backward_kernel<true><<<grid, flash_bwd::kThreads, flash_bwd::kSharedBytes, on>>>(
        k_map, v_map, q_map, do_map, dv_map, dk_map, workspace, seq, scale, causal ? 1u : 0u, device_status);
    FK_CUDA(cudaGetLastError());
    // Query-block owners: resident Q, dO; streamed K, V; output dQ (accumulator 1).
    flash_bwd::backward_kernel<false><<<grid, flash_bwd::kThreads, flash_bwd::kSharedBytes, on>>>(
        q_map, do_map, k_map, v_map, dq_map, dq_map, workspace, seq, scale, causal ? 1u : 0u, device_status);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}
