// Flash-attention forward, D = 128, for sm_100a:
//   O = softmax(scale * Q K^T [+ causal mask]) V,  bf16 in, fp32 softmax, bf16 (or fp32) out,
//   plus the fp32 log-sum-exp of every row.
//
// Replaces the reference kernel `flash_forward` and its launcher
// (examples/src/flash_forward.rs:150-310, 457-568), widened to a batch of planes,
// a non-causal mode, bf16 output and LSE. Same panel layout ([planes, seq, 128]
// bf16), same two contractions (Q K^T with both operands K-major; P V with V
// MN-major), same online softmax, output rows written by plain global stores like
// the reference's `store_rows` (src/global.rs:238-252). The structure is new: where
// the reference launches one CTA per query block and alternates MMA and softmax
// behind block-wide barriers, here one persistent CTA per SM walks a list of work
// items, each two 128-row query tiles that it ping-pongs, so the tensor core works
// on one tile while the CUDA cores run the other's softmax, and the next item's
// Q, first K block and first Q K^T overlap the current item's last softmax and
// read-out.
//
//   warps 0-7   softmax, one team of four warps per query tile (warps 0-3 tile 0, warps 4-7
//               tile 1), one thread per row: tcgen05.ld 32x32b of the row's 128 scores, running
//               max and sum in registers with no exchange between threads, P written back to
//               tensor memory as bf16 over S and published in two halves so that P.V starts under
//               the second half's exponentials; the output accumulator is rescaled in tensor
//               memory only when the max moved by more than 2^8; at the end of an item the team
//               reads its accumulator out, hands it back (`o_free`) and stores the normalised rows.
//               The two teams run independently, so one tile's exponentials overlap the other's
//               waits, loads and maxima on every scheduler.
//   warp 8      loader: per item Q_t as soon as the previous item's last Q K^T has read its
//               buffer, then K(j), V(j) 128-key blocks through a ring of kSlots slots that runs
//               on across items.
//   warp 9      MMA issue: S_t = Q_t K(j)^T (8 x M128 N128 K16) and O_t += P_t V(j)
//               (8 x M128 N128 K16, A from tensor memory), interleaved across the two tiles; the
//               next item's first S_t is issued right behind the current item's last P V.
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t
// aliases the first 64 columns of S_t. Causal launches skip key blocks above
// the diagonal, mask only the diagonal block, and pair a heavy query block with
// a light one of the same plane in every work item so that the items weigh the
// same. Barrier phases are carried across items. Every wait is bounded.

#include <mutex>

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
namespace flash {

constexpr uint32_t kTileRows = 128;   // query rows per tile
constexpr uint32_t kTiles = 2;        // query tiles per CTA
constexpr uint32_t kBlockKeys = 128;  // keys per K/V block
constexpr uint32_t kHead = 128;
constexpr uint32_t kSlots = 5;        // K/V ring depth, one [128, 128] bf16 block per slot
constexpr uint32_t kTeamWarps = 4;    // softmax warps per query tile: 32 rows each, one thread per row
constexpr uint32_t kSoftmaxWarps = kTeamWarps * kTiles;
constexpr uint32_t kLoaderWarp = kSoftmaxWarps;
constexpr uint32_t kMmaWarp = kSoftmaxWarps + 1;
// Three warpgroups: the two softmax teams, and one that holds the loader and the MMA warp (its
// other two warps idle). Registers are allocated per warpgroup, so the launch gives every thread
// kLaunchRegisters and the roles rebalance at once: a softmax thread holds its row's 128 scores
// and takes kSoftmaxRegisters, the third warpgroup keeps kServiceRegisters.
constexpr uint32_t kThreads = 3 * 128;
constexpr uint32_t kLaunchRegisters = 168;
constexpr uint32_t kSoftmaxRegisters = 200;
constexpr uint32_t kServiceRegisters = 104;
// setmaxnreg.inc waits until the pool holds the registers it asks for: the demands must fit what
// the launch allocated, or the wait never ends.
static_assert(kSoftmaxWarps * 32 * kSoftmaxRegisters + 128 * kServiceRegisters <= kThreads * kLaunchRegisters,
              "the warpgroups ask for more registers than the launch allocates");
static_assert(kThreads * kLaunchRegisters <= 65536, "the CTA's registers exceed the SM's register file");
constexpr uint32_t kSubtileBytes = 128 * 64 * 2;      // one [128, 64] bf16 SWIZZLE_128B subtile
constexpr uint32_t kBlockBytes = 2 * kSubtileBytes;   // one [128, 128] bf16 tile
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kScoreColumn = 0;     // S_t at kScoreColumn + 128 t
constexpr uint32_t kOutputColumn = 256;  // O_t at kOutputColumn + 128 t
// The running max is refreshed only when the block max exceeds it by this much (log2 domain).
constexpr float kRescaleThreshold = 8.0f;
// Of the 16 pairs of scores in a 32-column chunk, the pairs whose bit is set here take their
// 2^x from a polynomial on the FMA pipe instead of the ex2 unit: at D = 128 a score tile costs
// as many ex2-unit cycles as tensor cycles.
// Measured best share: four pairs of sixteen (three quarters of the exponentials stay on the unit).
constexpr uint32_t kPolyMask = 0x1111u;
// P is published in runs of 32-key chunks, each run on a barrier of its own: the P.V MMAs of a
// run are issued while the team is still exponentiating the runs after it. Bit c of the mask
// ends a run after chunk c (bit 3, the last chunk, always does).
// Two halves measured best (three quarters + one, and four quarters, lose 1-4 %: every run costs
// the team a tcgen05.wait::st).
constexpr uint32_t kPublishMask = 0xau;
static_assert((kPublishMask & 8u) && kPublishMask < 16u, "the last chunk ends the last run");
constexpr uint32_t kParts = ((kPublishMask >> 0) & 1u) + ((kPublishMask >> 1) & 1u) + ((kPublishMask >> 2) & 1u) + 1u;
// Run `part` covers chunks [run_first(part), run_first(part + 1)).
__host__ __device__ constexpr uint32_t run_first(uint32_t part) {
    uint32_t seen = 0;
    for (uint32_t c = 0; c < 4; ++c) {
        if (seen == part) return c;
        if ((kPublishMask >> c) & 1u) ++seen;
    }
    return 4;
}
__host__ __device__ constexpr uint32_t run_of(uint32_t chunk) {
    uint32_t part = 0;
    for (uint32_t c = 0; c < chunk; ++c)
        if ((kPublishMask >> c) & 1u) ++part;
    return part;
}

struct Plan {
    SharedPlan q, kv, q_full, q_empty, kv_full, kv_empty, s_full, p_ready, o_done, o_free, tmem_slot, stop, end;
    constexpr Plan()
        : q(SharedPlan{}.tile_ring(kTileRows, kHead, 2, kTiles)),
          kv(q.tile_ring(kBlockKeys, kHead, 2, kSlots)),
          q_full(kv.semaphores(kTiles)),
          q_empty(q_full.semaphores(kTiles)),
          kv_full(q_empty.semaphores(kSlots)),
          kv_empty(kv_full.semaphores(kSlots)),
          s_full(kv_empty.semaphores(kTiles)),
          p_ready(s_full.semaphores(kTiles * kParts)),
          o_done(p_ready.semaphores(kTiles)),
          o_free(o_done.semaphores(kTiles)),
          tmem_slot(o_free.tmem_slot()),
          stop(tmem_slot.word()),
          end(stop) {}
};
constexpr Plan kPlan{};
// Swizzled tiles need a 1024-byte-aligned base: the dynamic shared array is declared so, and
// the kernel refuses to run (status kMisaligned) should the base ever come back otherwise.
constexpr uint32_t kBaseAlign = 1024;
constexpr uint32_t kSharedBytes = static_cast<uint32_t>(kPlan.end.bytes());
static_assert(kSharedBytes <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");

enum StallCode : uint32_t {
    kStallLoader = 0x201,
    kStallMmaQ = 0x202,
    kStallMmaKv = 0x203,
    kStallMmaP = 0x204,
    kStallSoftmaxS = 0x205,
    kStallSoftmaxO = 0x206,
    kStallMmaOutput = 0x207,
    kStallLoaderQ = 0x208,
    kMisaligned = 0x2ff,
};

// What a launch hands every role so that each walks the same list of work items.
struct Problem {
    uint32_t seq;
    uint32_t planes;
    uint32_t pairs;   // query blocks of kTiles * kTileRows rows per plane: ceil(seq / 256)
    uint32_t causal;
    uint32_t whole;   // leading work items that are whole query blocks (two tiles)
    uint32_t items;   // entries the launch walks: `whole`, then the remaining blocks as two single tiles each
};

// One visit of a CTA: a query block of one plane, or nothing (`most` == 0).
struct Work {
    uint32_t plane;
    uint32_t q_row0;
    uint32_t blocks[kTiles];  // key blocks each query tile attends
    uint32_t most;
};

// Items of a launch, host and device: without a mask one query block each, plane-major, so that
// the CTAs running together share a plane's K and V through the L2. Under a causal mask a query
// block's work grows with its position, so an item is the pair {last - h, h} of one plane, heavy
// first: every item then weighs the same and a static round-robin over the CTAs is balanced.
__host__ __device__ __forceinline__ uint32_t item_count(uint32_t pairs, uint32_t planes, bool causal) {
    return (causal ? (pairs + 1) / 2 : pairs) * planes;
}

// The `visit`-th stop of CTA `cta` of `ctas`; false past the end of its list.
__device__ __forceinline__ bool work_at(const Problem& problem, uint32_t cta, uint32_t ctas, uint32_t visit,
                                        Work& work) {
    uint32_t q_block, single = 0, tiles = kTiles;
    bool present = true;
    if (problem.causal) {
        const uint32_t per_plane = (problem.pairs + 1) / 2;
        const uint32_t item = cta + (visit >> 1) * ctas;
        if (item >= problem.items) return false;
        const uint32_t h = item % per_plane;
        work.plane = item / per_plane;
        q_block = (visit & 1u) ? h : problem.pairs - 1 - h;
        present = !((visit & 1u) && h == problem.pairs - 1 - h);  // the middle block of an odd count, once
    } else {
        // The last, partly filled round of a launch is re-cut into single tiles when those still
        // fit one round: a tile alone takes about five sixths of a pair's time, and twice as many
        // CTAs share the round.
        const uint32_t entry = cta + visit * ctas;
        if (entry >= problem.items) return false;
        uint32_t item = entry;
        if (entry >= problem.whole) {
            const uint32_t rest = entry - problem.whole;
            item = problem.whole + (rest >> 1);
            single = rest & 1u;
            tiles = 1;
        }
        work.plane = item / problem.pairs;
        q_block = item % problem.pairs;
    }
    work.q_row0 = q_block * kTiles * kTileRows + kTileRows * single;
    work.most = 0;
    for (uint32_t t = 0; t < kTiles; ++t) {
        const uint32_t first = work.q_row0 + kTileRows * t;
        work.blocks[t] = (!present || t >= tiles || first >= problem.seq) ? 0u
                         : problem.causal                   ? first / kBlockKeys + 1u
                                                            : problem.seq / kBlockKeys;
        work.most = work.blocks[t] > work.most ? work.blocks[t] : work.most;
    }
    return true;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    // volatile: a fold must stay behind the tcgen05.wait::ld that makes its operands valid.
    asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ void st_global_v4(void* address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(address), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
    flash_forward_kernel(const __grid_constant__ CUtensorMap q_map,
                         const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map, uint16_t* __restrict__ o_bf16,
                         float* __restrict__ o_f32, float* __restrict__ lse, const Problem problem,
                         float scale, uint32_t* status) {
    extern __shared__ __align__(1024) uint8_t dynamic_shared[];
    const uint32_t base = smem_u32(dynamic_shared);
    if (base & (kBaseAlign - 1)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0u, static_cast<uint32_t>(kMisaligned));
        return;
    }

    const uint32_t q_tiles = base + kPlan.q.at;
    const uint32_t kv_ring = base + kPlan.kv.at;
    const uint32_t q_full = base + kPlan.q_full.at;
    const uint32_t q_empty = base + kPlan.q_empty.at;
    const uint32_t kv_full = base + kPlan.kv_full.at;
    const uint32_t kv_empty = base + kPlan.kv_empty.at;
    const uint32_t s_full = base + kPlan.s_full.at;
    const uint32_t p_ready = base + kPlan.p_ready.at;
    const uint32_t o_done = base + kPlan.o_done.at;
    const uint32_t o_free = base + kPlan.o_free.at;
    const uint32_t slot = base + kPlan.tmem_slot.at;
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.stop.at);
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.tmem_slot.at);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta = blockIdx.x, ctas = gridDim.x;
    const uint32_t seq = problem.seq;
    const bool causal = problem.causal != 0;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kSlots; ++s) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
        }
        for (uint32_t t = 0; t < kTiles; ++t) {
            mbar_init(q_full + 8 * t, 1);
            mbar_init(q_empty + 8 * t, 1);
            mbar_init(s_full + 8 * t, 1);
            for (uint32_t part = 0; part < kParts; ++part)
                mbar_init(p_ready + 8 * (kParts * t + part), kTeamWarps);
            mbar_init(o_done + 8 * t, 1);
            mbar_init(o_free + 8 * t, kTeamWarps);
        }
        *stop_flag = 0;
        fence_mbarrier_init();
        prefetch_tensormap(&q_map);
        prefetch_tensormap(&k_map);
        prefetch_tensormap(&v_map);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<1>(slot, kTmemColumns);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot_ptr;

    // The MMA thread sits on both tiles' dependency chains S -> softmax -> P -> P.V -> Q.K^T -> S
    // and polls: a thread suspended in try_wait comes back a few hundred cycles after the phase
    // completes. The softmax warps and the loader suspend: their probes would take issue slots
    // from the other team's warps on the same scheduler, and the kernel runs at the board's power
    // limit, where idle spinning is paid for in clock (measured: +2 % over everyone polling).
    const StallSite site_mma{status, stop_flag, 0, kWaitBudgetCycles, true};
    const StallSite site_softmax{status, stop_flag, 0, kWaitBudgetCycles, false};
    const StallSite site_loader{status, stop_flag, 0, kWaitBudgetCycles, false};

    // The rebalancing sits inside the role branches: ptxas budgets every instruction reachable
    // from a setmaxnreg by its count, so the two regions must not share code before the teardown.
    if (warp >= kSoftmaxWarps) {
      setmaxnreg_dec<kServiceRegisters>();
      if (warp == kLoaderWarp) {
        // ------------------------------------------------ loader
        if (lane == 0) {
            uint32_t fill = 0;               // K/V blocks put into the ring so far, all items
            uint32_t loaded[kTiles] = {0, 0};  // Q tiles loaded so far, per tile
            bool live = true;
            Work work;
            for (uint32_t visit = 0; live && work_at(problem, cta, ctas, visit, work); ++visit) {
                if (work.most == 0) continue;
                for (uint32_t t = 0; live && t < kTiles; ++t) {
                    if (!work.blocks[t]) continue;
                    // The previous item's last Q.K^T of this tile has read the buffer.
                    if (!mbar_wait(q_empty + 8 * t, (loaded[t] & 1u) ^ 1u, site_loader, kStallLoaderQ, loaded[t])) {
                        live = false;
                        break;
                    }
                    ++loaded[t];
                    mbar_arrive_expect_tx(q_full + 8 * t, kBlockBytes);
                    const int row = static_cast<int>(work.q_row0 + kTileRows * t);
                    for (uint32_t half = 0; half < 2; ++half)
                        tma_load_3d(q_tiles + t * kBlockBytes + half * kSubtileBytes, &q_map,
                                    static_cast<int>(64 * half), row, static_cast<int>(work.plane), q_full + 8 * t);
                }
                // Ring order: K(0), V(0), K(1), V(1), ...
                for (uint32_t i = 0; live && i < 2 * work.most; ++i, ++fill) {
                    const uint32_t s = fill % kSlots;
                    const uint32_t parity = (fill / kSlots) & 1u;
                    if (!mbar_wait(kv_empty + 8 * s, parity ^ 1u, site_loader, kStallLoader, fill)) {
                        live = false;
                        break;
                    }
                    mbar_arrive_expect_tx(kv_full + 8 * s, kBlockBytes);
                    const CUtensorMap* map = (i & 1u) ? &v_map : &k_map;
                    const int row = static_cast<int>(kBlockKeys * (i >> 1));
                    for (uint32_t half = 0; half < 2; ++half)
                        tma_load_3d(kv_ring + s * kBlockBytes + half * kSubtileBytes, map,
                                    static_cast<int>(64 * half), row, static_cast<int>(work.plane),
                                    kv_full + 8 * s);
                }
            }
        }
      } else if (warp == kMmaWarp) {
        // ------------------------------------------------ MMA issue
        // One thread issues, chosen by elect.sync: the compiler then knows the region runs in a
        // single thread (see the note at elect_one); chosen as lane 0 it does not.
        if (elect_one() != 0) {
            constexpr uint32_t idesc_qk = instruction_descriptor(kTileRows, kBlockKeys, false, false);
            constexpr uint32_t idesc_pv = instruction_descriptor(kTileRows, kHead, false, true);
            bool live = true;
            uint32_t started[kTiles] = {0, 0};  // items whose first Q.K^T was issued, per tile
            uint32_t blocks_done[kTiles] = {0, 0};  // P.V blocks issued so far, per tile, all items

            const auto wait_kv = [&](uint32_t fill) {
                if (!mbar_wait(kv_full + 8 * (fill % kSlots), (fill / kSlots) & 1u, site_mma, kStallMmaKv, fill)) {
                    live = false;
                    return false;
                }
                tc_fence_after_sync();
                return true;
            };
            // S_t = Q_t . K^T over d = 128: two stacked [128, 64] subtiles, four K=16 chunks each.
            const auto scores = [&](uint32_t t, uint32_t k_slot) {
                const uint32_t q_base = q_tiles + t * kBlockBytes;
                const uint32_t k_base = kv_ring + k_slot * kBlockBytes;
#pragma unroll
                for (uint32_t chunk = 0; chunk < kHead / 16; ++chunk) {
                    const uint32_t offset = (chunk / 4) * kSubtileBytes + (chunk % 4) * kKMajorChunkBytes;
                    mma_ss<1>(tmem + kScoreColumn + kBlockKeys * t,
                              operand_descriptor(q_base + offset, kKMajorLeadingBytes),
                              operand_descriptor(k_base + offset, kKMajorLeadingBytes), idesc_qk,
                              chunk != 0);
                }
                mma_commit<1>(s_full + 8 * t);
            };
            // O_t (+)= P_t . V over K=16 chunks [first, last) of the block: P from tensor memory
            // (8 columns per chunk), V MN-major: 16 key rows per chunk, the second 64 head
            // columns one subtile on.
            const auto output = [&](uint32_t t, uint32_t v_slot, bool accumulate, uint32_t first, uint32_t last) {
                const uint32_t v_base = kv_ring + v_slot * kBlockBytes;
#pragma unroll
                for (uint32_t chunk = first; chunk < last; ++chunk)
                    mma_ts(tmem + kOutputColumn + kHead * t,
                           tmem + kScoreColumn + kBlockKeys * t + 8 * chunk,
                           operand_descriptor(v_base + chunk * kMnMajorChunkBytes, kSubtileBytes),
                           idesc_pv, accumulate || chunk != 0);
            };
            // The first S_t of an item: its Q_t must have landed, its K(0) sits at ring position
            // `fill`. A tile with a single key block has read its Q for the last time here.
            const auto first_scores = [&](const Work& item, uint32_t t, uint32_t fill) {
                if (!mbar_wait(q_full + 8 * t, started[t] & 1u, site_mma, kStallMmaQ, started[t])) {
                    live = false;
                    return;
                }
                tc_fence_after_sync();
                ++started[t];
                scores(t, fill % kSlots);
                if (item.blocks[t] == 1) mma_commit<1>(q_empty + 8 * t);
            };

            Work work, next;
            uint32_t visit = 0;
            bool have = false;
            // The first item with work in it.
            while (work_at(problem, cta, ctas, visit, work)) {
                ++visit;
                if (work.most) {
                    have = true;
                    break;
                }
            }
            uint32_t fill = 0;  // ring position of K(0) of the current item
            if (have && wait_kv(fill)) {
                for (uint32_t t = 0; live && t < kTiles; ++t)
                    if (work.blocks[t]) first_scores(work, t, fill);
                if (live) mma_commit<1>(kv_empty + 8 * (fill % kSlots));
            }
            while (have && live) {
                bool have_next = false;
                while (work_at(problem, cta, ctas, visit, next)) {
                    ++visit;
                    if (next.most) {
                        have_next = true;
                        break;
                    }
                }
                const uint32_t next_fill = fill + 2 * work.most;
                for (uint32_t j = 0; live && j < work.most; ++j) {
                    const uint32_t v_use = fill + 2 * j + 1, k_use = fill + 2 * j + 2;
                    const uint32_t v_slot = v_use % kSlots, k_slot = k_use % kSlots;
                    const bool last = j + 1 == work.most;
                    if (!wait_kv(v_use)) break;
                    bool k_loaded = false;
                    for (uint32_t t = 0; live && t < kTiles; ++t) {
                        if (j < work.blocks[t]) {
                            if (j == 0) {
                                // The team has read the previous item's accumulator out.
                                if (!mbar_wait(o_free + 8 * t, (started[t] & 1u), site_mma, kStallMmaOutput, started[t])) {
                                    live = false;
                                    break;
                                }
                                tc_fence_after_sync();
                            }
#pragma unroll
                            for (uint32_t part = 0; part < kParts; ++part) {
                                if (!mbar_wait(p_ready + 8 * (kParts * t + part), blocks_done[t] & 1u, site_mma, kStallMmaP,
                                               blocks_done[t])) {
                                    live = false;
                                    break;
                                }
                                tc_fence_after_sync();
                                output(t, v_slot, j != 0, 2 * run_first(part), 2 * run_first(part + 1));
                            }
                            if (!live) break;
                            mma_commit<1>(o_done + 8 * t);
                            ++blocks_done[t];
                        }
                        if (j + 1 < work.blocks[t]) {
                            if (!k_loaded) {
                                if (!wait_kv(k_use)) break;
                                k_loaded = true;
                            }
                            scores(t, k_slot);
                            if (j + 2 == work.blocks[t]) mma_commit<1>(q_empty + 8 * t);  // Q_t's last reader
                        }
                        // Right behind this item's last P.V of the tile: the next item's first S_t.
                        if (last && have_next && next.blocks[t]) {
                            if (!k_loaded) {
                                if (!wait_kv(next_fill)) break;
                                k_loaded = true;
                            }
                            first_scores(next, t, next_fill);
                        }
                    }
                    if (!live) break;
                    mma_commit<1>(kv_empty + 8 * v_slot);
                    if (!last) mma_commit<1>(kv_empty + 8 * k_slot);
                    if (last && have_next) mma_commit<1>(kv_empty + 8 * (next_fill % kSlots));
                }
                fill = next_fill;
                work = next;
                have = have_next;
            }
        }
      }
    } else {
        setmaxnreg_inc<kSoftmaxRegisters>();
        // ------------------------------------------------ softmax, correction, read-out
        // One team of four warps per query tile, one thread per row: no value ever crosses
        // threads. The two teams share the four schedulers (warps w and w + 4 sit on the same
        // one) and are in different phases of their tiles, so one team's exponentials run while
        // the other waits for its next S, loads it and finds its maxima.
        const uint32_t t = warp / kTeamWarps;       // query tile of this team
        const uint32_t quadrant = warp & 3u;        // tensor-memory lanes this warp may touch
        const uint32_t row = 32 * quadrant + lane;  // row of the tile this thread owns
        const uint32_t lane_base = (32 * quadrant) << 16;
        const uint32_t s_tmem = tmem + lane_base + kScoreColumn + kBlockKeys * t;
        const uint32_t o_tmem = tmem + lane_base + kOutputColumn + kHead * t;
        const float scale_log2 = scale * 1.4426950408889634f;
        const float2 scale2 = make_float2(scale_log2, scale_log2);

        uint32_t g = 0;  // key blocks this team has seen, all items: the parity of its barriers
        bool live = true;
        Work work;
        for (uint32_t visit = 0; live && work_at(problem, cta, ctas, visit, work); ++visit) {
            const uint32_t blocks = work.blocks[t];
            if (blocks == 0) continue;
            float row_max = -INFINITY;  // raw score units
            float row_sum = 0.0f;

            for (uint32_t j = 0; live && j < blocks; ++j, ++g) {
                if (!mbar_wait(s_full + 8 * t, g & 1u, site_softmax, kStallSoftmaxS, g)) {
                    live = false;
                    break;
                }
                tc_fence_after_sync();
                uint32_t raw_s[4][32];
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) tmem_ld_32x32(s_tmem + 32 * c, raw_s[c]);
                tmem_wait_ld();

                if (causal && j + 1 == blocks) {
                    // Diagonal block: key (128 j + c) is visible to query (tile start + row) iff c <= row.
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c)
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i)
                            if (32 * c + i > row) raw_s[c][i] = 0xff800000u;  // -inf
                }

                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (uint32_t i = 0; i < 16; ++i) {
                    m0 = max3(m0, __uint_as_float(raw_s[0][2 * i]), __uint_as_float(raw_s[0][2 * i + 1]));
                    m1 = max3(m1, __uint_as_float(raw_s[1][2 * i]), __uint_as_float(raw_s[1][2 * i + 1]));
                    m2 = max3(m2, __uint_as_float(raw_s[2][2 * i]), __uint_as_float(raw_s[2][2 * i + 1]));
                    m3 = max3(m3, __uint_as_float(raw_s[3][2 * i]), __uint_as_float(raw_s[3][2 * i + 1]));
                }
                const float new_max = max3(row_max, fmaxf(m0, m1), fmaxf(m2, m3));
                const bool moved = (new_max - row_max) * scale_log2 > kRescaleThreshold;
                if (__any_sync(0xffffffffu, moved)) {
                    // Refresh this warp's maxima; rows whose max did not move scale by 1. A stale
                    // max is used consistently for P, the row sum and the log-sum-exp, so the
                    // result does not depend on when the refresh happens.
                    const float factor = ex2_approx((row_max - new_max) * scale_log2);
                    if (j > 0) {
                        if (!mbar_wait(o_done + 8 * t, (g - 1) & 1u, site_softmax, kStallSoftmaxO, g)) {
                            live = false;
                            break;
                        }
                        tc_fence_after_sync();
#pragma unroll 1
                        for (uint32_t c = 0; c < 4; ++c) {
                            uint32_t o[32];
                            tmem_ld_32x32(o_tmem + 32 * c, o);
                            tmem_wait_ld();
#pragma unroll
                            for (uint32_t i = 0; i < 32; ++i)
                                o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                            tmem_st_32x32(o_tmem + 32 * c, o);
                        }
                        tmem_wait_st();
                    }
                    row_sum *= factor;
                    row_max = new_max;
                }

                const float shift = row_max * scale_log2;
                const float2 shift2 = make_float2(-shift, -shift);
                // Four independent sum chains: with two, the compiler recycles the registers the
                // exponentials land in so tightly that every ex2 waits out the one before it and
                // the loop runs at half the unit's rate.
                float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
                float2 sum_c = make_float2(0.0f, 0.0f), sum_d = make_float2(0.0f, 0.0f);
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) {
                    // 32 keys -> 16 packed bf16 pairs, written over S columns this thread has read.
                    uint32_t packed[16];
#pragma unroll
                    for (uint32_t i = 0; i < 16; ++i) {
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw_s[c][2 * i]),
                                                                __uint_as_float(raw_s[c][2 * i + 1])),
                                                    scale2, shift2);
                        float2 p;
                        if ((kPolyMask >> i) & 1u) {
                            p = exp2_pair_fma(x);
                        } else {
                            p.x = ex2_approx(x.x);
                            p.y = ex2_approx(x.y);
                        }
                        if ((i & 3u) == 0)
                            sum_a = __fadd2_rn(sum_a, p);
                        else if ((i & 3u) == 1)
                            sum_b = __fadd2_rn(sum_b, p);
                        else if ((i & 3u) == 2)
                            sum_c = __fadd2_rn(sum_c, p);
                        else
                            sum_d = __fadd2_rn(sum_d, p);
                        packed[i] = pack_bf16x2(p.x, p.y);
                    }
                    tmem_st_32x16(s_tmem + 16 * c, packed);
                    if ((kPublishMask >> c) & 1u) {
                        if (c == 3)
                            row_sum += ((sum_a.x + sum_b.x) + (sum_c.x + sum_d.x)) +
                                       ((sum_a.y + sum_b.y) + (sum_c.y + sum_d.y));
                        tmem_wait_st();
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(p_ready + 8 * (kParts * t + run_of(c)));
                    }
                }
            }
            if (!live) break;

            // The item's last P.V has retired: read the accumulator out and store the rows.
            if (!mbar_wait(o_done + 8 * t, (g - 1) & 1u, site_softmax, kStallSoftmaxO, g)) {
                live = false;
                break;
            }
            tc_fence_after_sync();
            const float inverse = 1.0f / row_sum;
            const size_t q_index = static_cast<size_t>(work.plane) * seq + work.q_row0 + kTileRows * t + row;
            if (lse) lse[q_index] = (row_max * scale_log2 + lg2_approx(row_sum)) * 0.6931471805599453f;
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(o_tmem + 32 * c, o);
                tmem_wait_ld();
                if (c == 3) {
                    // Everything is in registers: the MMA thread may overwrite the accumulator.
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_free + 8 * t);
                }
                if (o_f32) {
                    float4* out = reinterpret_cast<float4*>(o_f32 + q_index * kHead + 32 * c);
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i)
                        out[i] = make_float4(__uint_as_float(o[4 * i]) * inverse,
                                             __uint_as_float(o[4 * i + 1]) * inverse,
                                             __uint_as_float(o[4 * i + 2]) * inverse,
                                             __uint_as_float(o[4 * i + 3]) * inverse);
                } else {
                    // A thread's row is 256 contiguous bytes of the output: 16-byte stores, every
                    // 32-byte sector written whole by two consecutive ones.
                    uint16_t* out = o_bf16 + q_index * kHead + 32 * c;
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t* v = o + 8 * i;
                        st_global_v4(out + 8 * i,
                                     pack_bf16x2(__uint_as_float(v[0]) * inverse, __uint_as_float(v[1]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[2]) * inverse, __uint_as_float(v[3]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[4]) * inverse, __uint_as_float(v[5]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[6]) * inverse, __uint_as_float(v[7]) * inverse));
                    }
                }
            }
        }
    }

    // ---------------------------------------------------- teardown
    if (*stop_flag) {
        // A role gave up: let copies and MMAs already in flight land before shared and tensor
        // memory are handed back.
        for (int i = 0; i < 256; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tmem_dealloc<1>(tmem, kTmemColumns);
}

}  // namespace flash
}  // namespace fk

// ------------------------------------------------------------------ C ABI

using namespace fk;

extern "C" uint32_t fk_flash_shared_bytes(void) { return flash::kSharedBytes; }
extern "C" uint32_t fk_flash_threads(void) { return flash::kThreads; }

extern "C" int fk_flash_fwd_launch(const void* q_map, const void* k_map, const void* v_map,
                                   void* o_bf16, float* o_f32, float* lse, uint32_t planes,
                                   uint32_t seq, float scale, int causal, void* stream,
                                   uint32_t* device_status) {
    if (!q_map || !k_map || !v_map) return fk_fail(FK_ERR_INVALID, "a tensor map pointer is null");
    if (!o_bf16 && !o_f32) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (seq == 0 || seq % flash::kTileRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE,
                       "%u queries x %u heads does not divide the %u queries a tile owns", seq,
                       planes, flash::kTileRows);
    if (reinterpret_cast<uintptr_t>(o_bf16) & 15u || reinterpret_cast<uintptr_t>(o_f32) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "the output wants 16-byte alignment");
    const uint32_t rows_per_item = flash::kTiles * flash::kTileRows;
    flash::Problem problem;
    problem.seq = seq;
    problem.planes = planes;
    problem.pairs = (seq + rows_per_item - 1) / rows_per_item;
    problem.causal = causal ? 1u : 0u;
    if (static_cast<uint64_t>(causal ? (problem.pairs + 1) / 2 : problem.pairs) * planes > 0x7fffffffull)
        return fk_fail(FK_ERR_SHAPE, "%u planes x %u queries is more work items than a launch walks", planes, seq);
    problem.items = problem.whole = flash::item_count(problem.pairs, planes, causal != 0);

    DeviceFacts facts;
    const int known = device_facts(&facts);
    if (known != FK_OK) return known;
    if (!causal) {
        // Items of one weight: what is left after the whole rounds goes out as single tiles when
        // two tiles per leftover block still fit one round of CTAs.
        const uint32_t round = static_cast<uint32_t>(facts.sm_count);
        const uint32_t tail = problem.items % round;
        if (tail != 0 && 2 * tail <= round) {
            problem.whole = problem.items - tail;
            problem.items = problem.whole + 2 * tail;
        }
    }
    uint32_t limit = 0;
    const int admitted = fk_admit_shared_plan(
        reinterpret_cast<const void*>(flash::flash_forward_kernel), flash::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;
    // One persistent CTA per SM (the plan and the 512 tensor-memory columns admit exactly one).
    const uint32_t sms = static_cast<uint32_t>(facts.sm_count);
    const dim3 grid(problem.items < sms ? problem.items : sms, 1, 1);
    flash::flash_forward_kernel<<<grid, flash::kThreads, flash::kSharedBytes,
                                  static_cast<cudaStream_t>(stream)>>>(
        *static_cast<const CUtensorMap*>(q_map), *static_cast<const CUtensorMap*>(k_map),
        *static_cast<const CUtensorMap*>(v_map), o_f32 ? nullptr : static_cast<uint16_t*>(o_bf16), o_f32, lse,
        problem, scale, device_status);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

extern "C" int fk_flash_fwd(const void* q, const void* k, const void* v, void* o_bf16, float* o_f32,
                            float* lse, uint32_t planes, uint32_t seq, float scale, int causal,
                            void* stream, uint32_t* device_status) {
    if (!q || !k || !v || (!o_bf16 && !o_f32))
        return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (seq == 0 || seq % flash::kTileRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE,
                       "%u queries x %u heads does not divide the %u queries a tile owns", seq,
                       planes, flash::kTileRows);
    alignas(64) CUtensorMap maps[3];
    int status = fk_encode_bf16_panels(&maps[0], reinterpret_cast<uint64_t>(q), flash::kTileRows,
                                       flash::kHead, seq, planes);
    if (status == FK_OK)
        status = fk_encode_bf16_panels(&maps[1], reinterpret_cast<uint64_t>(k), flash::kBlockKeys,
                                       flash::kHead, seq, planes);
    if (status == FK_OK)
        status = fk_encode_bf16_panels(&maps[2], reinterpret_cast<uint64_t>(v), flash::kBlockKeys,
                                       flash::kHead, seq, planes);
    if (status != FK_OK) return status;
    return fk_flash_fwd_launch(&maps[0], &maps[1], &maps[2], o_bf16, o_bf16 ? nullptr : o_f32, lse, planes, seq,
                               scale, causal, stream, device_status);
}

// One call at a time per device, like fk_gemm_bf16_host: the staging buffers and status words are
// the device's, so the call holds the device's guard until nothing of it is in flight.
extern "C" int fk_flash_fwd_host(const uint16_t* q_host, const uint16_t* k_host,
                                 const uint16_t* v_host, uint16_t* o_host, float* lse_host,
                                 uint32_t planes, uint32_t seq, float scale, int causal) {
    if (!q_host || !k_host || !v_host || !o_host)
        return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (seq == 0 || seq % flash::kTileRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE,
                       "%u queries x %u heads does not divide the %u queries a tile owns", seq,
                       planes, flash::kTileRows);
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> call(device_call_guard(device));
    const size_t bytes = size_t(planes) * seq * flash::kHead * 2;
    const size_t lse_bytes = size_t(planes) * seq * 4;
    void *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *lse = nullptr;
    uint32_t* status_words = nullptr;
    int status = scratch(3, bytes, &q);
    if (status == FK_OK) status = scratch(4, bytes, &k);
    if (status == FK_OK) status = scratch(5, bytes, &v);
    if (status == FK_OK) status = scratch(6, bytes, &o);
    if (status == FK_OK) status = scratch(7, lse_bytes, &lse);
    if (status == FK_OK) status = scratch_status(&status_words);
    if (status != FK_OK) return status;
    cudaStream_t stream = nullptr;
    const auto enqueue = [&]() -> int {
        FK_CUDA(cudaMemsetAsync(status_words, 0, 16, stream));
        FK_CUDA(cudaMemcpyAsync(q, q_host, bytes, cudaMemcpyHostToDevice, stream));
        FK_CUDA(cudaMemcpyAsync(k, k_host, bytes, cudaMemcpyHostToDevice, stream));
        FK_CUDA(cudaMemcpyAsync(v, v_host, bytes, cudaMemcpyHostToDevice, stream));
        const int launched = fk_flash_fwd(q, k, v, o, nullptr, static_cast<float*>(lse), planes, seq, scale,
                                          causal, stream, status_words);
        if (launched != FK_OK) return launched;
        FK_CUDA(cudaMemcpyAsync(o_host, o, bytes, cudaMemcpyDeviceToHost, stream));
        if (lse_host) FK_CUDA(cudaMemcpyAsync(lse_host, lse, lse_bytes, cudaMemcpyDeviceToHost, stream));
        return FK_OK;
    };
    status = enqueue();
    if (status != FK_OK) {
        wait_stream(stream);  // no copy of this call may still be reading the caller's buffers
        return status;
    }
    return fk_status_check(status_words, stream);
}
