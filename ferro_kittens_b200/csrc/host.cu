// Host surface behind the C ABI: global layouts and their tensor-map
// builders, the shared-plan cursor, the shared-memory opt-in, deadline waits
// and the device status decoder. Mirrors the host halves of the reference's
// `global` (src/global.rs:1649-2076), `plan` (src/plan.rs), `launch`
// (src/launch.rs) and `watchdog` (src/watchdog.rs) modules.

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <thread>

#include "fk_host.h"
#include "fk_layout.h"
#include "fk_ptx.cuh"

namespace fk {
constexpr int kMaxDevices = 64;
}

// ------------------------------------------------------------------ errors

static thread_local char fk_error_text[512] = "";

int fk_fail(int code, const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(fk_error_text, sizeof fk_error_text, format, args);
    va_end(args);
    return code;
}

extern "C" const char* fk_last_error(void) { return fk_error_text; }

// ------------------------------------------------------------------ layouts

static uint32_t element_bytes(uint32_t element) {
    switch (element) {
        case FK_BF16:
        case FK_F16:
            return 2;
        case FK_F32:
            return 4;
        default:
            return 0;
    }
}

static int layout_common(fk_layout_t* out, uint64_t base, uint32_t element, uint32_t rank,
                         const uint64_t* extents) {
    if (!out || !extents) return fk_fail(FK_ERR_INVALID, "a layout pointer is null");
    if (rank < 1 || rank > 5)
        return fk_fail(FK_ERR_INVALID, "cuTensorMapEncodeTiled describes rank 1 through 5");
    if (element_bytes(element) == 0) return fk_fail(FK_ERR_INVALID, "unknown element type %u", element);
    memset(out, 0, sizeof *out);
    out->base = base;
    out->rank = rank;
    out->element = element;
    for (uint32_t d = 0; d < rank; ++d) out->extents[d] = extents[d];
    return FK_OK;
}

extern "C" int fk_layout_packed(fk_layout_t* out, uint64_t base, uint32_t element, uint32_t rank,
                                const uint64_t* extents) {
    const int status = layout_common(out, base, element, rank, extents);
    if (status != FK_OK) return status;
    out->strides_bytes[0] = element_bytes(element);
    for (uint32_t d = 1; d < rank; ++d)
        out->strides_bytes[d] = out->strides_bytes[d - 1] * extents[d - 1];
    return FK_OK;
}

extern "C" int fk_layout_strided(fk_layout_t* out, uint64_t base, uint32_t element, uint32_t rank,
                                 const uint64_t* extents, const uint64_t* element_strides) {
    const int status = layout_common(out, base, element, rank, extents);
    if (status != FK_OK) return status;
    if (!element_strides) return fk_fail(FK_ERR_INVALID, "a layout pointer is null");
    if (element_strides[0] != 1)
        return fk_fail(FK_ERR_INVALID, "the TMA engine reads dimension 0 contiguously");
    for (uint32_t d = 0; d < rank; ++d)
        out->strides_bytes[d] = element_strides[d] * element_bytes(element);
    return FK_OK;
}

extern "C" int fk_layout_descriptor_shape(const fk_layout_t* layout, uint32_t box_columns,
                                          uint32_t box_rows, uint64_t* extents_out,
                                          uint32_t* box_out) {
    if (!layout || !extents_out || !box_out) return fk_fail(FK_ERR_INVALID, "a layout pointer is null");
    if (layout->rank == 1 && box_rows != 1)
        return fk_fail(FK_ERR_SHAPE, "a rank-1 layout has no dimension for a tile's rows");
    // Dimensions past the tile's own two select which box, one per instruction.
    for (uint32_t d = 0; d < layout->rank; ++d) {
        extents_out[d] = layout->extents[d];
        box_out[d] = 1;
    }
    box_out[0] = box_columns;
    if (layout->rank > 1) box_out[1] = box_rows;
    return FK_OK;
}

extern "C" int fk_layout_check(const fk_layout_t* layout, const uint64_t* extents,
                               const uint32_t* box) {
    if (!layout || !extents || !box) return fk_fail(FK_ERR_INVALID, "a layout pointer is null");
    if (layout->base % 16)
        return fk_fail(FK_ERR_ALIGNMENT, "tensor map base %#llx is not 16-byte aligned",
                       (unsigned long long)layout->base);
    for (uint32_t d = 1; d < layout->rank; ++d)
        if (layout->strides_bytes[d] % 16)
            return fk_fail(FK_ERR_ALIGNMENT,
                           "tensor map stride %llu of dimension %u is not a multiple of 16 bytes",
                           (unsigned long long)layout->strides_bytes[d], d);
    const uint64_t innermost = (uint64_t)box[0] * element_bytes(layout->element);
    if (innermost % 16)
        return fk_fail(FK_ERR_ALIGNMENT, "box dimension 0 is %llu bytes wide, not a multiple of 16",
                       (unsigned long long)innermost);
    for (uint32_t d = 0; d < layout->rank; ++d) {
        if (extents[d] < box[d])
            return fk_fail(FK_ERR_SHAPE, "dimension %u has extent %llu, smaller than its box %u", d,
                           (unsigned long long)extents[d], box[d]);
        if (box[d] > 256)
            return fk_fail(FK_ERR_SHAPE, "dimension %u has box %u, over the TMA maximum of 256", d,
                           box[d]);
    }
    return FK_OK;
}

// cuTensorMapEncodeTiled is reached through the runtime's driver entry point
// query, so the library links no driver stub and loads on a machine without one.
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_entry(EncodeTiled* out) {
    static std::mutex guard;
    static EncodeTiled cached = nullptr;
    std::lock_guard<std::mutex> lock(guard);
    if (!cached) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        FK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result));
        if (!entry || result != cudaDriverEntryPointSuccess)
            return fk_fail(FK_ERR_DRIVER, "the driver exports no cuTensorMapEncodeTiled");
        cached = reinterpret_cast<EncodeTiled>(entry);
    }
    *out = cached;
    return FK_OK;
}

extern "C" int fk_tensor_map(void* map_out, const fk_layout_t* layout, uint32_t box_columns,
                             uint32_t box_rows, uint32_t swizzle) {
    if (!map_out) return fk_fail(FK_ERR_INVALID, "a tensor map pointer is null");
    if ((uintptr_t)map_out % 64)
        return fk_fail(FK_ERR_ALIGNMENT, "a CUtensorMap must be 64-byte aligned");
    uint64_t extents[5];
    uint32_t box[5];
    int status = fk_layout_descriptor_shape(layout, box_columns, box_rows, extents, box);
    if (status != FK_OK) return status;
    status = fk_layout_check(layout, extents, box);
    if (status != FK_OK) return status;

    CUtensorMapDataType type;
    switch (layout->element) {
        case FK_BF16: type = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
        case FK_F16: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
        default: type = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    }
    CUtensorMapSwizzle mode;
    switch (swizzle) {
        case FK_SWIZZLE_NONE: mode = CU_TENSOR_MAP_SWIZZLE_NONE; break;
        case FK_SWIZZLE_128B: mode = CU_TENSOR_MAP_SWIZZLE_128B; break;
        default: return fk_fail(FK_ERR_INVALID, "unknown swizzle mode %u", swizzle);
    }
    EncodeTiled encode = nullptr;
    status = encode_entry(&encode);
    if (status != FK_OK) return status;
    // The driver call wants a context current on the calling thread; a thread that has made no
    // runtime call yet has none (the encode then fails with CUDA_ERROR_INVALID_CONTEXT). A null
    // free binds the device's primary context and does nothing else. Once per thread: the call is
    // not allowed while a stream of the thread is capturing, and a thread that captures has made
    // runtime calls before.
    static thread_local bool bound = false;
    if (!bound) {
        FK_CUDA(cudaFree(nullptr));
        bound = true;
    }

    cuuint64_t dims[5], strides[4];
    cuuint32_t boxes[5], element_strides[5];
    for (uint32_t d = 0; d < layout->rank; ++d) {
        dims[d] = extents[d];
        boxes[d] = box[d];
        element_strides[d] = 1;
        if (d > 0) strides[d - 1] = layout->strides_bytes[d];  // dimension 0's is implied
    }
    const CUresult result = encode(
        static_cast<CUtensorMap*>(map_out), type, layout->rank, reinterpret_cast<void*>(layout->base),
        dims, strides, boxes, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, mode,
        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS)
        return fk_fail(FK_ERR_DRIVER,
                       "cuTensorMapEncodeTiled(rank %u, extents [%llu, %llu, ..], box [%u, %u, ..]) "
                       "failed: %d",
                       layout->rank, (unsigned long long)extents[0],
                       (unsigned long long)(layout->rank > 1 ? extents[1] : 0), box[0],
                       layout->rank > 1 ? box[1] : 0, (int)result);
    return FK_OK;
}

extern "C" int fk_encode_bf16_panels(void* map_out, uint64_t base, uint32_t box_rows,
                                     uint32_t columns, uint64_t rows, uint64_t planes) {
    if (box_rows == 0 || rows % box_rows)
        return fk_fail(FK_ERR_SHAPE, "%llu rows is not a whole number of %u-row boxes",
                       (unsigned long long)rows, box_rows);
    const uint64_t extents[3] = {columns, rows, planes};
    fk_layout_t layout;
    const int status = fk_layout_packed(&layout, base, FK_BF16, 3, extents);
    if (status != FK_OK) return status;
    return fk_tensor_map(map_out, &layout, 64, box_rows, FK_SWIZZLE_128B);
}

// ------------------------------------------------------------------ plan

extern "C" void fk_plan_sizing(fk_plan_t* plan) {
    if (plan) plan->bytes = 0;
}
extern "C" uint64_t fk_plan_reserve(fk_plan_t* plan, uint64_t bytes, uint64_t align) {
    const fk::SharedPlan next = fk::SharedPlan{(size_t)plan->bytes, 0}.reserve(bytes, align);
    plan->bytes = next.bytes();
    return next.at;
}
extern "C" uint64_t fk_plan_tile(fk_plan_t* plan, uint32_t element, uint64_t rows, uint64_t columns) {
    return fk_plan_reserve(plan, rows * columns * element_bytes(element), fk::SharedPlan::kTileAlign);
}
extern "C" uint64_t fk_plan_tile_ring(fk_plan_t* plan, uint32_t element, uint64_t rows,
                                      uint64_t columns, uint64_t count) {
    return fk_plan_reserve(plan, rows * columns * element_bytes(element) * count,
                           fk::SharedPlan::kTileAlign);
}
extern "C" uint64_t fk_plan_semaphores(fk_plan_t* plan, uint64_t count) {
    return fk_plan_reserve(plan, count * fk::SharedPlan::kBarrierBytes, fk::SharedPlan::kBarrierAlign);
}
extern "C" uint64_t fk_plan_tmem_slot(fk_plan_t* plan) {
    return fk_plan_reserve(plan, fk::SharedPlan::kTmemSlotBytes, 4);
}

// ------------------------------------------------------------------ launch envelope

namespace fk {

int device_facts(DeviceFacts* out) {
    static std::mutex guard;
    static DeviceFacts known[64];
    static bool valid[64] = {};
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fk_fail(FK_ERR_INVALID, "device index %d out of range", device);
    std::lock_guard<std::mutex> lock(guard);
    if (!valid[device]) {
        DeviceFacts facts{device, 0, 0};
        FK_CUDA(cudaDeviceGetAttribute(&facts.sm_count, cudaDevAttrMultiProcessorCount, device));
        FK_CUDA(cudaDeviceGetAttribute(&facts.shared_optin_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        known[device] = facts;
        valid[device] = true;
    }
    *out = known[device];
    return FK_OK;
}

}  // namespace fk

// The admission is monotonic, so what has been granted to a (device, kernel) pair is remembered and a
// repeated request within it costs a table look-up instead of two runtime queries.
extern "C" int fk_admit_shared_plan(const void* kernel, uint32_t bytes, uint32_t* limit_out) {
    if (!kernel) return fk_fail(FK_ERR_INVALID, "the kernel pointer is null");
    fk::DeviceFacts facts;
    const int known = fk::device_facts(&facts);
    if (known != FK_OK) return known;
    const int limit = facts.shared_optin_limit;
    if (limit_out) *limit_out = (uint32_t)limit;
    if (bytes > (uint32_t)limit)
        return fk_fail(FK_ERR_TOO_LARGE,
                       "shared plan of %u B is past this device's %d B opt-in limit per block", bytes,
                       limit);
    struct Granted {
        const void* kernel;
        int device;
        uint32_t bytes;
    };
    static std::mutex guard;
    static Granted granted[64];
    static uint32_t count = 0;
    {
        std::lock_guard<std::mutex> lock(guard);
        for (uint32_t i = 0; i < count; ++i)
            if (granted[i].kernel == kernel && granted[i].device == facts.device && bytes <= granted[i].bytes)
                return FK_OK;
    }
    cudaFuncAttributes attributes;
    FK_CUDA(cudaFuncGetAttributes(&attributes, kernel));
    uint32_t now = (uint32_t)attributes.maxDynamicSharedSizeBytes;
    if (bytes > now) {  // never lowers
        FK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        now = bytes;
    }
    std::lock_guard<std::mutex> lock(guard);
    for (uint32_t i = 0; i < count; ++i)
        if (granted[i].kernel == kernel && granted[i].device == facts.device) {
            if (now > granted[i].bytes) granted[i].bytes = now;
            return FK_OK;
        }
    if (count < 64) granted[count++] = Granted{kernel, facts.device, now};
    return FK_OK;
}

// ------------------------------------------------------------------ arithmetic exports

extern "C" void fk_grouped(uint32_t item, uint32_t rows, uint32_t columns, uint32_t group,
                           uint32_t* row_out, uint32_t* column_out) {
    const fk::TileCoord tile = fk::grouped(item, rows, columns, group);
    *row_out = tile.row;
    *column_out = tile.column;
}
extern "C" uint32_t fk_swizzled_chunk_offset(uint32_t row, uint32_t chunk, uint32_t phase) {
    return fk::swizzled_chunk_offset(row, chunk, phase);
}
extern "C" uint64_t fk_operand_descriptor(uint64_t shared_address, uint32_t leading_bytes) {
    return fk::operand_descriptor(shared_address, leading_bytes);
}
extern "C" uint32_t fk_instruction_descriptor(uint32_t m, uint32_t n, int transpose_a,
                                              int transpose_b) {
    return fk::instruction_descriptor(m, n, transpose_a != 0, transpose_b != 0);
}
extern "C" uint32_t fk_tmem_address(uint32_t base, uint32_t row, uint32_t column) {
    return fk::tmem_address(base, row, column);
}

// ------------------------------------------------------------------ waits and status

// Spin for the first 50 ms (a launch's own length: be prompt), then sleep 1 ms between polls so
// that a wedged launch does not burn a core for the rest of its budget -- the reference's SPIN and
// POLL (src/watchdog.rs:117-121). Past the budget the reference ends the process; on a shared
// GPU this returns FK_ERR_TIMEOUT instead and leaves the decision to the caller.
template <typename Query>
static int poll_until(Query query, uint32_t budget_ms, const char* what) {
    const auto start = std::chrono::steady_clock::now();
    const auto budget = std::chrono::milliseconds(budget_ms);
    for (;;) {
        const cudaError_t status = query();
        if (status == cudaSuccess) return FK_OK;
        if (status != cudaErrorNotReady)
            return fk_fail(FK_ERR_DRIVER, "%s failed: %s", what, cudaGetErrorString(status));
        const auto waited = std::chrono::steady_clock::now() - start;
        if (waited >= budget)
            return fk_fail(FK_ERR_TIMEOUT, "%s still pending after %u ms (the launch deadline; %s overrides it)",
                           what, budget_ms, "KITTENS_LAUNCH_BUDGET_MS");
        if (waited >= std::chrono::milliseconds(50)) std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
}

extern "C" int fk_wait_stream(void* stream, uint32_t budget_ms) {
    return poll_until([&] { return cudaStreamQuery(static_cast<cudaStream_t>(stream)); }, budget_ms,
                      "cudaStreamQuery");
}
extern "C" int fk_wait_event(void* event, uint32_t budget_ms) {
    return poll_until([&] { return cudaEventQuery(static_cast<cudaEvent_t>(event)); }, budget_ms,
                      "cudaEventQuery");
}

// The budget every wait inside the library carries: the reference's 30 s default
// (src/watchdog.rs:102) unless its environment variable (:106) says otherwise. Read once, at the
// first wait, so that every wait of a run carries the same budget.
extern "C" uint32_t fk_launch_budget_ms(void) {
    static const uint32_t budget = [] {
        const char* text = getenv("KITTENS_LAUNCH_BUDGET_MS");
        if (text && *text) {
            char* end = nullptr;
            const unsigned long long value = strtoull(text, &end, 10);
            if (end && *end == '\0' && value > 0 && value <= 0xffffffffull) return static_cast<uint32_t>(value);
        }
        return 30000u;
    }();
    return budget;
}

// The deadline path without a device: a query that reports "not ready" `ready_after_polls` times
// (for ever when that is 0xffffffff) and then success, run through the same poll loop.
extern "C" int fk_selftest_deadline(uint32_t budget_ms, uint32_t ready_after_polls) {
    uint32_t polls = 0;
    return poll_until(
        [&] {
            if (ready_after_polls != 0xffffffffu && polls >= ready_after_polls) return cudaSuccess;
            ++polls;
            return cudaErrorNotReady;
        },
        budget_ms, "the self-test query");
}

extern "C" int fk_selftest_call_guard(int device, uint32_t hold_ms, uint64_t* entered_ns, uint64_t* left_ns) {
    if (device < 0 || device >= fk::kMaxDevices || !entered_ns || !left_ns)
        return fk_fail(FK_ERR_INVALID, "device index %d out of range or a null pointer", device);
    const auto now = [] {
        return static_cast<uint64_t>(std::chrono::duration_cast<std::chrono::nanoseconds>(
                                         std::chrono::steady_clock::now().time_since_epoch())
                                         .count());
    };
    std::lock_guard<std::mutex> call(fk::device_call_guard(device));
    *entered_ns = now();
    std::this_thread::sleep_for(std::chrono::milliseconds(hold_ms));
    *left_ns = now();
    return FK_OK;
}

namespace fk {

int wait_stream(cudaStream_t stream) { return fk_wait_stream(stream, fk_launch_budget_ms()); }

std::mutex& device_call_guard(int device) {
    static std::mutex guards[kMaxDevices];
    return guards[(device >= 0 && device < kMaxDevices) ? device : 0];
}

}  // namespace fk

static const char* stall_role(uint32_t code) {
    switch (code) {
        case 0x101: return "gemm producer waiting for a free stage";
        case 0x102: return "gemm MMA waiting for a loaded stage";
        case 0x103: return "gemm MMA waiting for a drained accumulator";
        case 0x104: return "gemm epilogue waiting for a finished accumulator";
        case 0x105: return "gemm role waiting for the item feed";
        case 0x106: return "gemm item feed waiting for the answer to a cluster-launch-control request";
        case 0x201: return "flash loader waiting for a free K/V slot";
        case 0x202: return "flash MMA waiting for Q";
        case 0x203: return "flash MMA waiting for a loaded K/V slot";
        case 0x204: return "flash MMA waiting for P";
        case 0x205: return "flash softmax waiting for S";
        case 0x206: return "flash softmax waiting for O";
        case 0x207: return "flash MMA waiting for the previous item's output to be read out";
        case 0x208: return "flash loader waiting for a free Q buffer";
        case 0x1ff: return "gemm found its shared memory base off a 1024-byte boundary";
        case 0x2ff: return "flash found its shared memory base off a 1024-byte boundary";
        case 0x301: return "self-test wait on a barrier nothing arrives on";
        case 0x401: return "flash backward loader waiting for a free ring stage";
        case 0x402: return "flash backward MMA warp waiting for its resident tiles";
        case 0x403: return "flash backward MMA warp waiting for a streamed block";
        case 0x404: return "flash backward MMA warp waiting for P and dS";
        case 0x405: return "flash backward element-wise warp waiting for S and dP";
        case 0x406: return "flash backward element-wise warp waiting for the accumulators";
        case 0x407: return "flash backward MMA warp waiting for dS";
        case 0x408: return "flash backward element-wise warp waiting for dP";
        case 0x4ff: return "flash backward found its shared memory base off a 1024-byte boundary";
        case 0x312: return "row-kernel copy warp waiting for the compute warps to finish a tile";
        case 0x313: return "row-kernel compute warp waiting for a tile to land";
        case 0x314: return "row-kernel compute warp waiting for the other warps' partial sums";
        default: return "unknown role";
    }
}

extern "C" int fk_status_check(const uint32_t* device_status, void* stream) {
    if (!device_status) return FK_OK;
    uint32_t words[4] = {0, 0, 0, 0};
    FK_CUDA(cudaMemcpyAsync(words, device_status, sizeof words, cudaMemcpyDeviceToHost,
                            static_cast<cudaStream_t>(stream)));
    const int waited = fk::wait_stream(static_cast<cudaStream_t>(stream));
    if (waited != FK_OK) return waited;
    if (words[0] == 0) return FK_OK;
    return fk_fail(FK_ERR_DEVICE_STALL, "device stall: %s (code %#x) in block %u, step %u, parity %u",
                   stall_role(words[0]), words[0], words[1], words[2], words[3]);
}

// A wait that nothing will ever complete, with a short budget: exercises the bounded-wait,
// status-word and clean-exit path that both kernels rely on, without starving any barrier that
// real data depends on. The kernel returns normally and the context stays usable.
__global__ void stall_probe_kernel(uint32_t* status, long long budget_cycles) {
    __shared__ __align__(8) unsigned long long barrier;
    __shared__ uint32_t stop;
    const uint32_t bar = fk::smem_u32(&barrier);
    if (threadIdx.x == 0) {
        fk::mbar_init(bar, 1);
        stop = 0;
        fk::fence_mbarrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const fk::StallSite site{status, &stop, 0, budget_cycles};
        fk::mbar_wait(bar, 0, site, 0x301, 7);
    }
    __syncthreads();
    if (threadIdx.x == 0) fk::mbar_inval(bar);
}

// The FMA-pipe 2^x the attention kernels use for a share of their exponentials, alone: y[i] = 2^x[i]
// for pairs of inputs, so that a test can hold it to the bound the reference states for its own
// `exp2_approx` (src/reg.rs:81-93, test :2047-2062).
__global__ void exp2_probe_kernel(const float2* x, float2* y, uint32_t pairs) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < pairs) y[i] = fk::exp2_pair_fma(x[i]);
}

extern "C" int fk_selftest_exp2(const float* x, float* y, uint32_t count, void* stream) {
    if (!x || !y || count % 2) return fk_fail(FK_ERR_INVALID, "null pointer or an odd number of values");
    const uint32_t pairs = count / 2;
    if (pairs == 0) return FK_OK;
    exp2_probe_kernel<<<(pairs + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const float2*>(x), reinterpret_cast<float2*>(y), pairs);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

extern "C" int fk_selftest_stall(void* stream, uint32_t* device_status, uint32_t budget_cycles) {
    if (!device_status) return fk_fail(FK_ERR_INVALID, "the status pointer is null");
    stall_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_status, budget_cycles);
    FK_CUDA(cudaGetLastError());
    return FK_OK;
}

// ------------------------------------------------------------------ per-device scratch

namespace fk {

constexpr int kSlots = 8;
static std::mutex scratch_guard;
static void* scratch_base[kMaxDevices][kSlots];
static size_t scratch_size[kMaxDevices][kSlots];
static uint32_t* status_words[kMaxDevices];

int scratch(int slot, size_t bytes, void** out) {
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    if (device >= kMaxDevices || slot >= kSlots) return fk_fail(FK_ERR_INVALID, "scratch slot out of range");
    std::lock_guard<std::mutex> lock(scratch_guard);
    if (scratch_size[device][slot] < bytes) {
        // Callers hold the device's call guard and leave nothing in flight behind their return, so
        // no kernel or copy can still be using the buffer that is replaced here.
        if (scratch_base[device][slot]) FK_CUDA(cudaFree(scratch_base[device][slot]));
        scratch_base[device][slot] = nullptr;
        scratch_size[device][slot] = 0;
        FK_CUDA(cudaMalloc(&scratch_base[device][slot], bytes));
        scratch_size[device][slot] = bytes;
    }
    *out = scratch_base[device][slot];
    return FK_OK;
}

int scratch_status(uint32_t** out) {
    int device = 0;
    FK_CUDA(cudaGetDevice(&device));
    if (device >= kMaxDevices) return fk_fail(FK_ERR_INVALID, "device index out of range");
    std::lock_guard<std::mutex> lock(scratch_guard);
    if (!status_words[device]) FK_CUDA(cudaMalloc(&status_words[device], 8 * sizeof(uint32_t)));
    *out = status_words[device];
    return FK_OK;
}

}  // namespace fk
