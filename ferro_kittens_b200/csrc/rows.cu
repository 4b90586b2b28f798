// The memory-bound row kernels that sit either side of attention and GEMM in a transformer
// block, for sm_100a: row-wise base-2 softmax, layernorm over rows, and the whole-tile
// normalisation, over rows of 128 bf16 columns.
//
// They replace the reference's `softmax_rows` (examples/src/softmax.rs:105-186),
// `layernorm_rows` and `groupnorm_tile` (examples/src/layernorm.rs:125-306): same arithmetic in
// the same order (fp32 in registers, one rounding to bf16 on the way out), same [128, 128] tile
// as the unit the whole-tile statistic is taken over. The structure is new. The reference
// launches one CTA per tile, which loads, computes and stores in sequence; here one persistent
// CTA per SM streams its tiles through a ring of kStages shared-memory slots:
//
//   warp 16     lane 0 issues a bulk copy (cp.async.bulk, 32 KiB: a tile is 128 whole rows and so
//               contiguous in global memory) per tile, kStages - 1 tiles ahead of the compute
//               warps, and the bulk store of each finished tile from the same slot;
//   warps 0-15  8 rows of the tile each: 16 lanes per row, 16 bytes (8 columns) per lane, the
//               whole tile share (32 values per lane) in registers, reductions by shuffles inside
//               the half-warp, results written back over the slot in place.
//
// HBM is the roofline: 4 bytes per element (2 in, 2 out). Three tiles (96 KiB) are in flight per SM;
// deeper rings measured slower (5.5-5.9 TB/s at six slots against 6.2-6.6 at four). Every wait is bounded.

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
namespace rows {

constexpr uint32_t kTileRows = 128;
constexpr uint32_t kColumns = 128;
constexpr uint32_t kRowBytes = kColumns * 2;
constexpr uint32_t kTileBytes = kTileRows * kRowBytes;  // 32 KiB
constexpr uint32_t kStages = 4;
constexpr uint32_t kComputeWarps = 16;
constexpr uint32_t kWarpRows = kTileRows / kComputeWarps;  // 8
constexpr uint32_t kSteps = kWarpRows / 2;                 // two rows per warp-wide access
constexpr uint32_t kThreads = (kComputeWarps + 1) * 32;

enum Operation : int { kSoftmax = 0, kLayerNorm = 1, kGroupNorm = 2 };

struct Plan {
    SharedPlan ring, full, done, agree, partials, stop, end;
    constexpr Plan()
        : ring(SharedPlan{}.reserve(kStages * kTileBytes, 128)),
          full(ring.semaphores(kStages)),
          done(full.semaphores(kStages)),
          agree(done.semaphores(2)),
          partials(agree.reserve(2 * kComputeWarps * 4, 16)),
          stop(partials.word()),
          end(stop) {}
};
constexpr Plan kPlan{};
constexpr uint32_t kSharedBytes = static_cast<uint32_t>(kPlan.end.bytes());
static_assert(kSharedBytes <= 232448, "plan exceeds the opt-in shared memory of an sm_100 CTA");

enum StallCode : uint32_t {
    kStallLoad = 0x311,     // producer waiting for a slot's store to finish reading (not a barrier)
    kStallStore = 0x312,    // producer waiting for the compute warps to finish a tile
    kStallCompute = 0x313,  // compute warp waiting for a tile to land
    kStallAgree = 0x314,    // compute warp waiting for the other warps' partial sums
};

struct Arguments {
    const uint8_t* source;
    uint8_t* destination;
    const uint16_t* gamma;
    const uint16_t* beta;
    uint32_t tiles;
    float epsilon;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t (&v)[4]) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
// Sum over the 16 lanes that hold one row.
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
    for (uint32_t mask = 8; mask > 0; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
    return v;
}

// Element-wise maximum of two packed bf16 pairs.
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

template <int OP>
__global__ void __launch_bounds__(kThreads, 1) rows_kernel(const Arguments args, uint32_t* status) {
    extern __shared__ __align__(128) uint8_t dynamic_shared[];
    const uint32_t base = smem_u32(dynamic_shared);
    const uint32_t ring = base + kPlan.ring.at;
    const uint32_t full = base + kPlan.full.at;
    const uint32_t done = base + kPlan.done.at;
    const uint32_t agree = base + kPlan.agree.at;
    float* const partials = reinterpret_cast<float*>(dynamic_shared + kPlan.partials.at);
    volatile uint32_t* stop_flag = reinterpret_cast<volatile uint32_t*>(dynamic_shared + kPlan.stop.at);

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    // This CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...
    const uint32_t count = args.tiles > blockIdx.x ? (args.tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full + 8 * s, 1);
            mbar_init(done + 8 * s, kComputeWarps);
        }
        mbar_init(agree, kComputeWarps);
        mbar_init(agree + 8, kComputeWarps);
        *stop_flag = 0;
        fence_mbarrier_init();
    }
    __syncthreads();
    const StallSite site{status, stop_flag, 0};

    if (warp == kComputeWarps) {
        // ------------------------------------------------ copies in and out
        if (lane == 0) {
            constexpr uint32_t kLead = kStages - 1;
            for (uint32_t it = 0; it < count + kLead; ++it) {
                if (it >= kLead) {
                    // The tile loaded kLead iterations ago is finished: store it from its slot.
                    const uint32_t j = it - kLead, s = j % kStages;
                    if (!mbar_wait(done + 8 * s, (j / kStages) & 1u, site, kStallStore, j)) break;
                    const size_t tile = blockIdx.x + static_cast<size_t>(j) * gridDim.x;
                    bulk_store(args.destination + tile * kTileBytes, ring + s * kTileBytes, kTileBytes);
                    tma_store_commit();
                }
                if (it < count) {
                    // Slot it % kStages last held tile it - kStages, whose store was committed one
                    // iteration ago; only the store committed just above may still be reading.
                    tma_store_wait_read<1>();
                    const uint32_t s = it % kStages;
                    const size_t tile = blockIdx.x + static_cast<size_t>(it) * gridDim.x;
                    mbar_arrive_expect_tx(full + 8 * s, kTileBytes);
                    bulk_load(ring + s * kTileBytes, args.source + tile * kTileBytes, kTileBytes, full + 8 * s);
                }
            }
            tma_store_wait_before_exit();
        }
    } else {
        // ------------------------------------------------ arithmetic
        const uint32_t sub = lane >> 4;    // which of the two rows of a step
        const uint32_t chunk = lane & 15;  // which 8 columns of the row
        const uint32_t offset = (kWarpRows * warp + sub) * kRowBytes + chunk * 16;
        // Everything below works on packed fp32 pairs (add/mul/fma.f32x2): half the instructions of
        // the scalar form, which is what keeps these kernels on the memory roofline when the chip
        // runs at its power-capped clock.
        float2 gamma[4], beta[4];
        if (OP == kLayerNorm) {
            const uint4 g = *reinterpret_cast<const uint4*>(args.gamma + 8 * chunk);
            const uint4 b = *reinterpret_cast<const uint4*>(args.beta + 8 * chunk);
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                gamma[i] = make_float2(__uint_as_float(gw[i] << 16), __uint_as_float(gw[i] & 0xffff0000u));
                beta[i] = make_float2(__uint_as_float(bw[i] << 16), __uint_as_float(bw[i] & 0xffff0000u));
            }
        }
        uint32_t agreements = 0;
        // All compute warps fold their partial sums: a bounded rendezvous, alternating two barriers
        // and two halves of the scratch so that a fast warp's next use cannot overtake a slow one's read.
        auto tile_sum = [&](float value, bool& live) {
#pragma unroll
            for (uint32_t mask = 16; mask > 0; mask >>= 1) value += __shfl_xor_sync(0xffffffffu, value, mask);
            const uint32_t which = agreements & 1u;
            if (lane == 0) partials[which * kComputeWarps + warp] = value;
            __syncwarp();
            if (lane == 0) mbar_arrive(agree + 8 * which);
            if (!mbar_wait(agree + 8 * which, (agreements >> 1) & 1u, site, kStallAgree, agreements)) live = false;
            ++agreements;
            float total = 0.0f;
#pragma unroll
            for (uint32_t w = 0; w < kComputeWarps; ++w) total += partials[which * kComputeWarps + w];
            return total;
        };
        // Sum of the eight values a lane holds of one row.
        const auto lane_sum = [](const float2 (&v)[4]) {
            const float2 pair = __fadd2_rn(__fadd2_rn(v[0], v[1]), __fadd2_rn(v[2], v[3]));
            return pair.x + pair.y;
        };

        bool live = true;
        for (uint32_t it = 0; live && it < count; ++it) {
            const uint32_t s = it % kStages;
            if (!mbar_wait(full + 8 * s, (it / kStages) & 1u, site, kStallCompute, it)) break;
            const uint32_t slot = ring + s * kTileBytes + offset;
            float2 x[kSteps][4];
            uint32_t words[kSteps][4];
#pragma unroll
            for (uint32_t step = 0; step < kSteps; ++step) {
                ld_shared_v4(slot + step * 2 * kRowBytes, words[step]);
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i)
                    x[step][i] = make_float2(__uint_as_float(words[step][i] << 16),
                                             __uint_as_float(words[step][i] & 0xffff0000u));
            }

            if (OP == kSoftmax) {
                // 2^(x - peak) / sum, the reference's three passes (softmax.rs:137-160) over registers.
                // The peak is found on the packed bf16 words: the maximum of bf16 values is one of them.
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step) {
                    uint32_t top = max_bf16x2(max_bf16x2(words[step][0], words[step][1]),
                                              max_bf16x2(words[step][2], words[step][3]));
#pragma unroll
                    for (uint32_t mask = 8; mask > 0; mask >>= 1)
                        top = max_bf16x2(top, __shfl_xor_sync(0xffffffffu, top, mask));
                    const float peak = fmaxf(__uint_as_float(top << 16), __uint_as_float(top & 0xffff0000u));
                    const float2 shift = make_float2(-peak, -peak);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        const float2 d = __fadd2_rn(x[step][i], shift);
                        x[step][i] = make_float2(ex2_approx(d.x), ex2_approx(d.y));
                    }
                    const float scale = __frcp_rn(row_sum(lane_sum(x[step])));
                    const float2 scale2 = make_float2(scale, scale);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) x[step][i] = __fmul2_rn(x[step][i], scale2);
                }
            } else if (OP == kLayerNorm) {
                // Mean, centred variance, then gamma * (x - mean) * rsqrt(var + eps) + beta
                // (layernorm.rs:173-206).
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step) {
                    const float mean = row_sum(lane_sum(x[step])) * (1.0f / kColumns);
                    const float2 shift = make_float2(-mean, -mean);
                    float2 square = make_float2(0.0f, 0.0f);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        x[step][i] = __fadd2_rn(x[step][i], shift);
                        square = __ffma2_rn(x[step][i], x[step][i], square);
                    }
                    const float deviation = rsqrtf(row_sum(square.x + square.y) * (1.0f / kColumns) + args.epsilon);
                    const float2 deviation2 = make_float2(deviation, deviation);
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i)
                        x[step][i] = __ffma2_rn(__fmul2_rn(x[step][i], deviation2), gamma[i], beta[i]);
                }
            } else {
                // The same statistic over the whole tile (layernorm.rs:262-300).
                constexpr float kScale = 1.0f / (kTileRows * kColumns);
                float2 total = make_float2(0.0f, 0.0f);
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step)
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) total = __fadd2_rn(total, x[step][i]);
                const float mean = tile_sum(total.x + total.y, live) * kScale;
                if (!live) break;
                const float2 shift = make_float2(-mean, -mean);
                float2 square = make_float2(0.0f, 0.0f);
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step)
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        x[step][i] = __fadd2_rn(x[step][i], shift);
                        square = __ffma2_rn(x[step][i], x[step][i], square);
                    }
                const float deviation = rsqrtf(tile_sum(square.x + square.y, live) * kScale + args.epsilon);
                if (!live) break;
                const float2 deviation2 = make_float2(deviation, deviation);
#pragma unroll
                for (uint32_t step = 0; step < kSteps; ++step)
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) x[step][i] = __fmul2_rn(x[step][i], deviation2);
            }

#pragma unroll
            for (uint32_t step = 0; step < kSteps; ++step)
                st_shared_v4(slot + step * 2 * kRowBytes, pack_bf16x2(x[step][0].x, x[step][0].y),
                             pack_bf16x2(x[step][1].x, x[step][1].y), pack_bf16x2(x[step][2].x, x[step][2].y),
                             pack_bf16x2(x[step][3].x, x[step][3].y));
            // The bulk store reads the slot through the async proxy.
            fence_proxy_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive(done + 8 * s);
        }
    }
}

}  // namespace rows
}  // namespace fk

// ------------------------------------------------------------------ C ABI

using namespace fk;

extern "C" uint32_t fk_rows_shared_bytes(void) { return rows::kSharedBytes; }
extern "C" uint32_t fk_rows_threads(void) { return rows::kThreads; }

template <int OP>
static int launch_rows(const void* source, const void* gamma, const void* beta, void* destination,
                       uint64_t rows_total, float epsilon, void* stream, uint32_t* device_status) {
    if (!source || !destination) return fk_fail(FK_ERR_INVALID, "an operand pointer is null");
    if (OP == rows::kLayerNorm && (!gamma || !beta))
        return fk_fail(FK_ERR_INVALID, "a parameter vector pointer is null");
    if ((reinterpret_cast<uintptr_t>(source) | reinterpret_cast<uintptr_t>(destination) |
         reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(beta)) & 15u)
        return fk_fail(FK_ERR_ALIGNMENT, "bulk copies want 16-byte aligned buffers");
    if (rows_total / rows::kTileRows > 0xffffffffull)
        return fk_fail(FK_ERR_SHAPE, "%llu rows is more tiles than a launch counts",
                       static_cast<unsigned long long>(rows_total));
    DeviceFacts facts;
    const int known = device_facts(&facts);
    if (known != FK_OK) return known;
    const int sm_count = facts.sm_count;
    uint32_t limit = 0;
    const int admitted =
        fk_admit_shared_plan(reinterpret_cast<const void*>(rows::rows_kernel<OP>), rows::kSharedBytes, &limit);
    if (admitted != FK_OK) return admitted;
    rows::Arguments args;
    args.source = static_cast<const uint8_t*>(source);
    args.destination = static_cast<uint8_t*>(destination);
    args.gamma = static_cast<const uint16_t*>(gamma);
    args.beta = static_cast<const uint16_t*>(beta);
    args.tiles = static_cast<uint32_t>(rows_total / rows::kTileRows);
    args.epsilon = epsilon;
    const uint32_t grid = args.tiles < static_cast<uint32_t>(sm_count) ? args.tiles : static_cast<uint32_t>(sm_count);
    rows::rows_kernel<OP><<<grid, rows::kThreads, rows::kSharedBytes, static_cast<cudaStream_t>(stream)>>>(
        args, device_status);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

extern "C" int fk_softmax_rows(const void* source, void* destination, uint32_t rows_per_plane,
                               uint32_t planes, void* stream, uint32_t* device_status) {
    if (rows_per_plane == 0 || rows_per_plane % rows::kTileRows || planes == 0)
        return fk_fail(FK_ERR_SHAPE, "%u rows x %u planes does not divide %u rows a CTA", rows_per_plane,
                       planes, rows::kTileRows);
    return launch_rows<rows::kSoftmax>(source, nullptr, nullptr, destination,
                                       static_cast<uint64_t>(rows_per_plane) * planes, 0.0f, stream,
                                       device_status);
}

extern "C" int fk_layernorm_rows(const void* source, const void* gamma, const void* beta,
                                 void* destination, uint32_t row_count, float epsilon, void* stream,
                                 uint32_t* device_status) {
    if (row_count == 0 || row_count % rows::kTileRows)
        return fk_fail(FK_ERR_SHAPE, "%u rows does not divide the %u a CTA owns", row_count, rows::kTileRows);
    return launch_rows<rows::kLayerNorm>(source, gamma, beta, destination, row_count, epsilon, stream,
                                         device_status);
}

extern "C" int fk_groupnorm_tile(const void* source, void* destination, uint32_t row_count,
                                 float epsilon, void* stream, uint32_t* device_status) {
    if (row_count == 0 || row_count % rows::kTileRows)
        return fk_fail(FK_ERR_SHAPE, "%u rows does not divide the %u a CTA owns", row_count, rows::kTileRows);
    return launch_rows<rows::kGroupNorm>(source, nullptr, nullptr, destination, row_count, epsilon, stream,
                                         device_status);
}
