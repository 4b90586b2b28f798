// Flash-attention forward, D = 128, for sm_100a:
//   O = softmax(scale * Q K^T [+ causal mask]) V,  bf16 in, fp32 softmax, bf16 (or fp32) out,
//   plus the fp32 log-sum-exp of every row.
//
// Replaces the reference kernel `flash_forward` and its launcher
// (examples/src/flash_forward.rs:150-310, 457-568), widened to a batch of planes,
// a non-causal mode, bf16 output and LSE. Same panel layout ([planes, seq, 128]
// bf16), same two contractions (Q K^T with both operands K-major; P V with V
// MN-major), same online softmax. The structure is new: where the reference
// alternates MMA and softmax behind block-wide barriers, one CTA here owns two
// 128-row query tiles and ping-pongs them, so the tensor core works on one
// tile while the CUDA cores run the other's softmax.
//
//   warps 0-7   softmax, one team of four warps per query tile (warps 0-3 tile 0, warps 4-7
//               tile 1), one thread per row: tcgen05.ld 32x32b of the row's 128 scores, running
//               max and sum in registers with no exchange between threads, P written back to
//               tensor memory as bf16 over S and published in two halves so that P.V starts under
//               the second half's exponentials; the output accumulator is rescaled in tensor
//               memory only when the max moved by more than 2^8; final normalise, bf16 staging
//               and TMA store. The two teams run independently, so one tile's exponentials
//               overlap the other's waits, loads and maxima on every scheduler.
//   warp 8      loader: Q once, then K(j), V(j) 128-key blocks through a ring of kSlots slots.
//   warp 9      MMA issue: S_t = Q_t K(j)^T (8 x M128 N128 K16) and O_t += P_t V(j)
//               (8 x M128 N128 K16, A from tensor memory), interleaved across the two tiles.
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P_t
// aliases the first 64 columns of S_t. Causal launches skip key blocks above
// the diagonal and mask only the diagonal block. Every wait is bounded.

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
constexpr uint32_t kSoftmaxRegisters = 208;
constexpr uint32_t kServiceRegisters = 88;
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
#ifndef FK_FLASH_POLY_MASK
#define FK_FLASH_POLY_MASK 0x1111u
#endif
constexpr uint32_t kPolyMask = FK_FLASH_POLY_MASK;
// P is published in two halves of 64 keys: the first four P.V MMAs of a block are issued while
// the team is still exponentiating the second half.
#ifndef FK_FLASH_SPLIT
#define FK_FLASH_SPLIT 1
#endif
constexpr bool kSplitPublish = FK_FLASH_SPLIT != 0;

struct Plan {
    SharedPlan q, kv, q_full, kv_full, kv_empty, s_full, p_half, p_ready, o_done, tmem_slot, stop, end;
    constexpr Plan()
        : q(SharedPlan{}.tile_ring(kTileRows, kHead, 2, kTiles)),
          kv(q.tile_ring(kBlockKeys, kHead, 2, kSlots)),
          q_full(kv.semaphore()),
          kv_full(q_full.semaphores(kSlots)),
          kv_empty(kv_full.semaphores(kSlots)),
          s_full(kv_empty.semaphores(kTiles)),
          p_half(s_full.semaphores(kTiles)),
          p_ready(p_half.semaphores(kTiles)),
          o_done(p_ready.semaphores(kTiles)),
          tmem_slot(o_done.tmem_slot()),
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
    kMisaligned = 0x2ff,
};

struct Extent {
    uint32_t blocks[kTiles];  // key blocks each query tile attends
    uint32_t most;
};

// Key blocks per tile: all of them, or up to and including the diagonal block.
__device__ __forceinline__ Extent extent(uint32_t q_row0, uint32_t seq, bool causal) {
    Extent e;
    e.most = 0;
    for (uint32_t t = 0; t < kTiles; ++t) {
        const uint32_t first = q_row0 + kTileRows * t;
        e.blocks[t] = first >= seq ? 0u : (causal ? first / kBlockKeys + 1u : seq / kBlockKeys);
        e.most = e.blocks[t] > e.most ? e.blocks[t] : e.most;
    }
    return e;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__global__ void __launch_bounds__(kThreads, 1)
    flash_forward_kernel(const __grid_constant__ CUtensorMap q_map,
                         const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map,
                         const __grid_constant__ CUtensorMap o_map, float* __restrict__ o_f32,
                         float* __restrict__ lse, uint32_t seq, float scale, uint32_t causal,
                         uint32_t* status) {
    extern __shared__ __align__(1024) uint8_t dynamic_shared[];
    const uint32_t base = smem_u32(dynamic_shared);
    if (base & (kBaseAlign - 1)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0u, static_cast<uint32_t>(kMisaligned));
        return;
    }

    const uint32_t q_tiles = base + kPlan.q.at;
    const uint32_t kv_ring = base + kPlan.kv.at;
    const uint32_t q_full = base + kPlan.q_full.at;
    const uint32_t kv_full = base + kPlan.kv_full.at;
    const uint32_t kv_empty = base + kPlan.kv_empty.at;
    const uint32_t s_full = base + kPlan.s_full.at;
    const uint32_t p_half = base + kPlan.p_half.at;
    const uint32_t p_ready = base + kPlan.p_ready.at;
    const uint32_t o_done = base + kPlan.o_done.at;
    const uint32_t slot = base + kPlan.tmem_slot.at;
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.stop.at);
    volatile uint32_t* slot_ptr = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.tmem_slot.at);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t plane = blockIdx.y;
    // Causal work grows with the query block: launch the heaviest CTAs first.
    const uint32_t q_block = causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x;
    const uint32_t q_row0 = q_block * kTiles * kTileRows;
    const Extent keys = extent(q_row0, seq, causal != 0);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (uint32_t s = 0; s < kSlots; ++s) {
            mbar_init(kv_full + 8 * s, 1);
            mbar_init(kv_empty + 8 * s, 1);
        }
        for (uint32_t t = 0; t < kTiles; ++t) {
            mbar_init(s_full + 8 * t, 1);
            mbar_init(p_half + 8 * t, kTeamWarps);
            mbar_init(p_ready + 8 * t, kTeamWarps);
            mbar_init(o_done + 8 * t, 1);
        }
        *stop_flag = 0;
        fence_mbarrier_init();
        prefetch_tensormap(&q_map);
        prefetch_tensormap(&k_map);
        prefetch_tensormap(&v_map);
        prefetch_tensormap(&o_map);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<1>(slot, kTmemColumns);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot_ptr;

    // Every role here sits on a tile's dependency chain S -> softmax -> P -> P.V -> Q.K^T -> S:
    // a thread suspended in try_wait comes back a few hundred cycles after the phase completes,
    // so the roles poll instead (measured: +2.5 to +3.8 %).
    const StallSite site{status, stop_flag, 0, kWaitBudgetCycles, true};

    // The rebalancing sits inside the role branches: ptxas budgets every instruction reachable
    // from a setmaxnreg by its count, so the two regions must not share code before the teardown.
    if (warp >= kSoftmaxWarps) {
      setmaxnreg_dec<kServiceRegisters>();
      if (warp == kLoaderWarp) {
        // ------------------------------------------------ loader
        if (lane == 0) {
            uint32_t q_bytes = 0;
            for (uint32_t t = 0; t < kTiles; ++t) q_bytes += keys.blocks[t] ? kBlockBytes : 0u;
            mbar_arrive_expect_tx(q_full, q_bytes);
            for (uint32_t t = 0; t < kTiles; ++t) {
                if (!keys.blocks[t]) continue;
                const int row = static_cast<int>(q_row0 + kTileRows * t);
                for (uint32_t half = 0; half < 2; ++half)
                    tma_load_3d(q_tiles + t * kBlockBytes + half * kSubtileBytes, &q_map,
                                static_cast<int>(64 * half), row, static_cast<int>(plane), q_full);
            }
            // Ring order: K(0), V(0), K(1), V(1), ...
            for (uint32_t fill = 0; fill < 2 * keys.most; ++fill) {
                const uint32_t s = fill % kSlots;
                const uint32_t parity = (fill / kSlots) & 1u;
                if (!mbar_wait(kv_empty + 8 * s, parity ^ 1u, site, kStallLoader, fill)) break;
                mbar_arrive_expect_tx(kv_full + 8 * s, kBlockBytes);
                const CUtensorMap* map = (fill & 1u) ? &v_map : &k_map;
                const int row = static_cast<int>(kBlockKeys * (fill >> 1));
                for (uint32_t half = 0; half < 2; ++half)
                    tma_load_3d(kv_ring + s * kBlockBytes + half * kSubtileBytes, map,
                                static_cast<int>(64 * half), row, static_cast<int>(plane),
                                kv_full + 8 * s);
            }
        }
      } else if (warp == kMmaWarp) {
        // ------------------------------------------------ MMA issue
        // One thread issues, chosen by elect.sync: the compiler then knows the region runs in a
        // single thread (see the note at elect_one); chosen as lane 0 it does not.
        if (elect_one() != 0) {
            constexpr uint32_t idesc_qk = instruction_descriptor(kTileRows, kBlockKeys, false, false);
            constexpr uint32_t idesc_pv = instruction_descriptor(kTileRows, kHead, false, true);

            // S_t = Q_t . K^T over d = 128: two stacked [128, 64] subtiles, four K=16 chunks each.
            auto scores = [&](uint32_t t, uint32_t k_slot) {
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
            // O_t (+)= P_t . V over keys [16 first, 16 last) of the block: P from tensor memory
            // (8 columns per K=16 chunk), V MN-major: 16 key rows per chunk, the second 64 head
            // columns one subtile on.
            auto output = [&](uint32_t t, uint32_t v_slot, bool accumulate, uint32_t first, uint32_t last) {
                const uint32_t v_base = kv_ring + v_slot * kBlockBytes;
#pragma unroll
                for (uint32_t chunk = first; chunk < last; ++chunk)
                    mma_ts(tmem + kOutputColumn + kHead * t,
                           tmem + kScoreColumn + kBlockKeys * t + 8 * chunk,
                           operand_descriptor(v_base + chunk * kMnMajorChunkBytes, kSubtileBytes),
                           idesc_pv, accumulate || chunk != 0);
            };
            constexpr uint32_t kChunks = kBlockKeys / 16;

            bool live = mbar_wait(q_full, 0, site, kStallMmaQ, 0);
            if (live) {
                tc_fence_after_sync();
                live = mbar_wait(kv_full + 0, 0, site, kStallMmaKv, 0);
            }
            if (live) {
                tc_fence_after_sync();
                for (uint32_t t = 0; t < kTiles; ++t)
                    if (keys.blocks[t]) scores(t, 0);
                mma_commit<1>(kv_empty + 0);
            }
            for (uint32_t j = 0; live && j < keys.most; ++j) {
                const uint32_t v_use = 2 * j + 1, k_use = 2 * j + 2;
                const uint32_t v_slot = v_use % kSlots, k_slot = k_use % kSlots;
                const bool more = j + 1 < keys.most;
                if (!mbar_wait(kv_full + 8 * v_slot, (v_use / kSlots) & 1u, site, kStallMmaKv, v_use))
                    break;
                bool next_loaded = false;
                for (uint32_t t = 0; live && t < kTiles; ++t) {
                    if (j < keys.blocks[t]) {
                        if (kSplitPublish) {
                            if (!mbar_wait(p_half + 8 * t, j & 1u, site, kStallMmaP, j)) {
                                live = false;
                                break;
                            }
                            tc_fence_after_sync();
                            output(t, v_slot, j != 0, 0, kChunks / 2);
                        }
                        if (!mbar_wait(p_ready + 8 * t, j & 1u, site, kStallMmaP, j)) {
                            live = false;
                            break;
                        }
                        tc_fence_after_sync();
                        output(t, v_slot, j != 0, kSplitPublish ? kChunks / 2 : 0, kChunks);
                        mma_commit<1>(o_done + 8 * t);
                    }
                    if (j + 1 < keys.blocks[t]) {
                        if (!next_loaded) {
                            if (!mbar_wait(kv_full + 8 * k_slot, (k_use / kSlots) & 1u, site,
                                           kStallMmaKv, k_use)) {
                                live = false;
                                break;
                            }
                            tc_fence_after_sync();
                            next_loaded = true;
                        }
                        scores(t, k_slot);
                    }
                }
                if (!live) break;
                mma_commit<1>(kv_empty + 8 * v_slot);
                if (more) mma_commit<1>(kv_empty + 8 * k_slot);
            }
        }
      }
    } else {
        setmaxnreg_inc<kSoftmaxRegisters>();
        // ------------------------------------------------ softmax, correction, epilogue
        // One team of four warps per query tile, one thread per row: no value ever crosses
        // threads. The two teams share the four schedulers (warps w and w + 4 sit on the same
        // one) and are in different phases of their tiles, so one team's exponentials run while
        // the other waits for its next S, loads it and finds its maxima.
        const uint32_t t = warp / kTeamWarps;       // query tile of this team
        const uint32_t quadrant = warp & 3u;        // tensor-memory lanes this warp may touch
        const uint32_t row = 32 * quadrant + lane;  // row of the tile this thread owns
        const uint32_t blocks = keys.blocks[t];
        const uint32_t lane_base = (32 * quadrant) << 16;
        const uint32_t s_tmem = tmem + lane_base + kScoreColumn + kBlockKeys * t;
        const uint32_t o_tmem = tmem + lane_base + kOutputColumn + kHead * t;
        const float scale_log2 = scale * 1.4426950408889634f;
        const float2 scale2 = make_float2(scale_log2, scale_log2);

        float row_max = -INFINITY;  // raw score units
        float row_sum = 0.0f;
        bool live = blocks != 0;

        for (uint32_t j = 0; live && j < blocks; ++j) {
            if (!mbar_wait(s_full + 8 * t, j & 1u, site, kStallSoftmaxS, j)) {
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
                // max is used consistently for P, the row sum and the log-sum-exp, so the result
                // does not depend on when the refresh happens.
                const float factor = ex2_approx((row_max - new_max) * scale_log2);
                if (j > 0) {
                    if (!mbar_wait(o_done + 8 * t, (j - 1) & 1u, site, kStallSoftmaxO, j)) {
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
                if (kSplitPublish && c == 1) {
                    tmem_wait_st();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(p_half + 8 * t);
                }
            }
            row_sum += ((sum_a.x + sum_b.x) + (sum_c.x + sum_d.x)) + ((sum_a.y + sum_b.y) + (sum_c.y + sum_d.y));
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready + 8 * t);
        }

        if (live) live = mbar_wait(o_done + 8 * t, (blocks - 1) & 1u, site, kStallSoftmaxO, blocks);
        if (live) {
            tc_fence_after_sync();
            const float inverse = 1.0f / row_sum;
            const uint32_t q_index = q_row0 + kTileRows * t + row;
            if (lse)
                lse[static_cast<size_t>(plane) * seq + q_index] =
                    (row_max * scale_log2 + lg2_approx(row_sum)) * 0.6931471805599453f;
            // Q_t's shared tile is dead once the last MMA retired: it stages the output. This
            // warp owns rows [32 q, 32 q + 32) of both [128, 64] subtiles.
            const uint32_t stage = q_tiles + t * kBlockBytes;
#pragma unroll 1
            for (uint32_t c = 0; c < 4; ++c) {
                uint32_t o[32];
                tmem_ld_32x32(o_tmem + 32 * c, o);
                tmem_wait_ld();
                if (o_f32) {
                    float4* out = reinterpret_cast<float4*>(
                        o_f32 + (static_cast<size_t>(plane) * seq + q_index) * kHead + 32 * c);
#pragma unroll
                    for (uint32_t i = 0; i < 8; ++i)
                        out[i] = make_float4(__uint_as_float(o[4 * i]) * inverse,
                                             __uint_as_float(o[4 * i + 1]) * inverse,
                                             __uint_as_float(o[4 * i + 2]) * inverse,
                                             __uint_as_float(o[4 * i + 3]) * inverse);
                } else {
                    const uint32_t subtile = stage + (c / 2) * kSubtileBytes;
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const uint32_t* v = o + 8 * i;
                        st_shared_v4(subtile + swizzled_chunk_offset(row, 4 * (c % 2) + i, 0),
                                     pack_bf16x2(__uint_as_float(v[0]) * inverse,
                                                 __uint_as_float(v[1]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[2]) * inverse,
                                                 __uint_as_float(v[3]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[4]) * inverse,
                                                 __uint_as_float(v[5]) * inverse),
                                     pack_bf16x2(__uint_as_float(v[6]) * inverse,
                                                 __uint_as_float(v[7]) * inverse));
                    }
                }
            }
            if (!o_f32) {
                fence_proxy_async_shared();
                __syncwarp();
                if (lane == 0) {
                    const int out_row = static_cast<int>(q_row0 + kTileRows * t + 32 * quadrant);
                    for (uint32_t half = 0; half < 2; ++half)
                        tma_store_3d(&o_map, stage + half * kSubtileBytes + 32 * quadrant * 128,
                                     static_cast<int>(64 * half), out_row, static_cast<int>(plane));
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_before_exit();
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
                                   const void* o_map, float* o_f32, float* lse, uint32_t planes,
                                   uint32_t seq, float scale, int causal, void* stream,
                                   uint32_t* device_status) {
    if (!q_map || !k_map || !v_map || (!o_map && !o_f32))
        return fk_fail(FK_ERR_INVALID, "a tensor map pointer is null");
    if (seq == 0 || seq % flash::kTileRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE,
                       "%u queries x %u heads does not divide the %u queries a tile owns", seq,
                       planes, flash::kTileRows);
    if (planes > 65535) return fk_fail(FK_ERR_SHAPE, "%u planes is past the 65535 a launch takes", planes);
    uint32_t limit = 0;
    const int admitted = fk_admit_shared_plan(
        reinterpret_cast<const void*>(flash::flash_forward_kernel), flash::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;
    const uint32_t rows_per_cta = flash::kTiles * flash::kTileRows;
    const dim3 grid((seq + rows_per_cta - 1) / rows_per_cta, planes, 1);
    const CUtensorMap* store = static_cast<const CUtensorMap*>(o_map ? o_map : q_map);
    flash::flash_forward_kernel<<<grid, flash::kThreads, flash::kSharedBytes,
                                  static_cast<cudaStream_t>(stream)>>>(
        *static_cast<const CUtensorMap*>(q_map), *static_cast<const CUtensorMap*>(k_map),
        *static_cast<const CUtensorMap*>(v_map), *store, o_f32, lse, seq, scale, causal ? 1u : 0u,
        device_status);
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
    alignas(64) CUtensorMap maps[4];
    int status = fk_encode_bf16_panels(&maps[0], reinterpret_cast<uint64_t>(q), flash::kTileRows,
                                       flash::kHead, seq, planes);
    if (status == FK_OK)
        status = fk_encode_bf16_panels(&maps[1], reinterpret_cast<uint64_t>(k), flash::kBlockKeys,
                                       flash::kHead, seq, planes);
    if (status == FK_OK)
        status = fk_encode_bf16_panels(&maps[2], reinterpret_cast<uint64_t>(v), flash::kBlockKeys,
                                       flash::kHead, seq, planes);
    if (status == FK_OK && o_bf16)
        status = fk_encode_bf16_panels(&maps[3], reinterpret_cast<uint64_t>(o_bf16), 32, flash::kHead,
                                       seq, planes);
    if (status != FK_OK) return status;
    return fk_flash_fwd_launch(&maps[0], &maps[1], &maps[2], o_bf16 ? &maps[3] : nullptr,
                               o_bf16 ? nullptr : o_f32, lse, planes, seq, scale, causal, stream,
                               device_status);
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
