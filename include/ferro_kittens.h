/*
 * ferro_kittens.h -- C ABI of the B200 (sm_100a) implementation of ferro-kittens'
 * two dense-contraction hot paths: the two-CTA-cluster bf16 GEMM and
 * flash-attention forward.
 *
 * Every entry point is what a Rust `extern "C"` block in the ferro-kittens crate
 * would bind to keep its host surface (`global`, `plan`, `launch`, `watchdog`,
 * the two kernel entry points) while the kernels behind it are CUDA C++.
 * Each declaration cites the reference item it stands in for, by the file's
 * path inside the ferro-kittens repository.
 *
 * Conventions: plain pointers and sizes only; device pointers are `void*` /
 * `const void*`; a `cudaStream_t` is passed as `void*`; a tensor map is the
 * driver's 128-byte, 64-byte-aligned `CUtensorMap`, owned by the caller and
 * passed by address (the kernels take it by value as a grid constant, so no
 * device upload is needed). Functions return FK_OK or a negative error code;
 * `fk_last_error()` returns the thread-local message naming the violated field.
 * Nothing here falls back to a CPU path.
 */
#ifndef FERRO_KITTENS_H
#define FERRO_KITTENS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FK_OK = 0,
    FK_ERR_INVALID = -1,      /* null pointer / bad enum */
    FK_ERR_SHAPE = -2,        /* shape does not divide the tiling, zero group, ... */
    FK_ERR_ALIGNMENT = -3,    /* a driver alignment rule of the tensor map */
    FK_ERR_TOO_LARGE = -4,    /* shared plan past the device's opt-in limit */
    FK_ERR_DRIVER = -5,       /* the CUDA driver / runtime refused a call */
    FK_ERR_TIMEOUT = -6,      /* a host wait ran out of its budget */
    FK_ERR_DEVICE_STALL = -7  /* a kernel's bounded wait gave up; see fk_status_check */
};

typedef enum { FK_BF16 = 0, FK_F16 = 1, FK_F32 = 2 } fk_element_t;
typedef enum { FK_SWIZZLE_NONE = 0, FK_SWIZZLE_128B = 3 } fk_swizzle_t;

/* Thread-local message of the last failing call on this thread ("" if none). */
const char* fk_last_error(void);

/* ---------------------------------------------------------------- global layouts
 *
 * `GlobalLayout<E, RANK>` (src/global.rs:1767-1889): a RANK-dimensional buffer,
 * dimension 0 contiguous; `strides_bytes[0]` is the element size and is implied
 * to the driver. `fk_layout_packed` = `GlobalLayout::packed` (:1794-1802),
 * `fk_layout_strided` = `GlobalLayout::strided` (:1826-1841; fails unless
 * element_strides[0] == 1).
 */
typedef struct {
    uint64_t base;             /* device address; never dereferenced on the host */
    uint32_t rank;             /* 1..5 */
    uint32_t element;          /* fk_element_t */
    uint64_t extents[5];       /* dimension 0 fastest */
    uint64_t strides_bytes[5]; /* byte stride of each dimension */
} fk_layout_t;

int fk_layout_packed(fk_layout_t* out, uint64_t base, uint32_t element, uint32_t rank,
                     const uint64_t* extents);
int fk_layout_strided(fk_layout_t* out, uint64_t base, uint32_t element, uint32_t rank,
                      const uint64_t* extents, const uint64_t* element_strides);

/* `GlobalLayout::descriptor_shape::<T>` (src/global.rs:1867-1888): globalDim and
 * boxDim for a map delivering a tile whose box is [box_columns, box_rows]. */
int fk_layout_descriptor_shape(const fk_layout_t* layout, uint32_t box_columns, uint32_t box_rows,
                               uint64_t* extents_out, uint32_t* box_out);

/* `GlobalLayout::check_driver_requirements` (src/global.rs:1969-2017): base 16-byte
 * aligned, strides multiples of 16, box dimension 0 a multiple of 16 bytes, no box
 * wider than its extent, no box over 256. Needs no driver. */
int fk_layout_check(const fk_layout_t* layout, const uint64_t* extents, const uint32_t* box);

/* `GlobalLayout::tensor_map::<T>` (src/global.rs:1920-1964) over
 * cuTensorMapEncodeTiled: element strides 1, INTERLEAVE_NONE, the given swizzle,
 * L2 promotion NONE, OOB fill NONE. `map_out` is 128 bytes, 64-byte aligned. */
int fk_tensor_map(void* map_out, const fk_layout_t* layout, uint32_t box_columns,
                  uint32_t box_rows, uint32_t swizzle);

/* `encode_bf16_panels::<R, C>` (src/global.rs:2067-2076): rank-3 SWIZZLE_128B map
 * over a packed [planes, rows, columns] bf16 buffer, box [64, box_rows, 1];
 * fails unless rows % box_rows == 0. */
int fk_encode_bf16_panels(void* map_out, uint64_t base, uint32_t box_rows, uint32_t columns,
                          uint64_t rows, uint64_t planes);

/* ---------------------------------------------------------------- plan / launch
 *
 * `SharedPlan` (src/plan.rs:73-304) as a cursor of two words. Each reservation
 * aligns to its own rule (tiles 128, barriers 8, slot 4) and returns the start
 * of the run; `bytes` is what a launch declares.
 */
typedef struct {
    uint64_t bytes;
} fk_plan_t;

void fk_plan_sizing(fk_plan_t* plan);                                        /* :143-150 */
uint64_t fk_plan_reserve(fk_plan_t* plan, uint64_t bytes, uint64_t align);   /* :177-195 */
uint64_t fk_plan_tile(fk_plan_t* plan, uint32_t element, uint64_t rows, uint64_t columns);
uint64_t fk_plan_tile_ring(fk_plan_t* plan, uint32_t element, uint64_t rows, uint64_t columns,
                           uint64_t count);                                  /* :213-225 */
uint64_t fk_plan_semaphores(fk_plan_t* plan, uint64_t count);                /* :263-267 */
uint64_t fk_plan_tmem_slot(fk_plan_t* plan);                                 /* :276-279 */

/* Dynamic shared memory the two kernels declare (the `#[launch_contract]`
 * literal of examples/src/gemm.rs:397-402 and SHARED_BYTES of
 * examples/src/flash_forward.rs:141, for this implementation's own plans). */
uint32_t fk_gemm_shared_bytes(void);
uint32_t fk_gemm_threads(void);
uint32_t fk_flash_shared_bytes(void);
uint32_t fk_flash_threads(void);

/* `gemm::grid` (examples/src/gemm.rs:472-475): CTAs of a launch resident at a time, a whole
 * number of two-CTA clusters, capped at one cluster per SM pair. (A launch of more items than
 * that puts one cluster per item in its grid; the resident clusters never exit and take the
 * others' items over one by one through cluster launch control, so the items in flight are always
 * the next ones of the traversal.) */
uint32_t fk_gemm_grid(uint32_t m, uint32_t n, uint32_t sm_count);

/* `launch::admit_shared_plan` (src/launch.rs:110-132): opt `kernel` (a host
 * function pointer of a __global__) into `bytes` of dynamic shared memory.
 * Idempotent, never lowers; FK_ERR_TOO_LARGE past the device's opt-in limit,
 * which is written to `limit_out` either way. */
int fk_admit_shared_plan(const void* kernel, uint32_t bytes, uint32_t* limit_out);

/* ---------------------------------------------------------------- traversal and descriptors
 * Pure arithmetic, exported so a binding's tests can pin it without a GPU. */
void fk_grouped(uint32_t item, uint32_t rows, uint32_t columns, uint32_t group, uint32_t* row_out,
                uint32_t* column_out);                     /* src/pipeline.rs:207-213 */
uint32_t fk_swizzled_chunk_offset(uint32_t row, uint32_t chunk, uint32_t phase);
                                                           /* src/shared.rs:1341-1348 */
uint64_t fk_operand_descriptor(uint64_t shared_address, uint32_t leading_bytes);
                                                           /* src/shared.rs:1251-1258 */
uint32_t fk_instruction_descriptor(uint32_t m, uint32_t n, int transpose_a, int transpose_b);
                                                           /* src/mma.rs:137-146 */
uint32_t fk_tmem_address(uint32_t base, uint32_t row, uint32_t column); /* src/tmem.rs:487 */

/* ---------------------------------------------------------------- kernels
 *
 * GEMM: `kernels::gemm_cg2_staged_x8x4` + `gemm::run`'s guards
 * (examples/src/gemm.rs:404-413, 487-496). C[m,n] = sum_k A[m,k]*B[n,k]; A is
 * row-major [m,k] bf16, B is K-major [n,k] bf16, C row-major [m,n] bf16.
 *   a_map: rank-2 dims [k, m], box [64, 128], SWIZZLE_128B
 *   b_map: rank-2 dims [k, n], box [64, 128], SWIZZLE_128B
 *   c_map: rank-2 dims [n, m] (outer stride = ldc bytes), box [64, 32], SWIZZLE_128B
 * Requires m % 256 == 0, n % 256 == 0, k % 64 == 0, group >= 1. Asynchronous on
 * `stream`. `device_status` is null or 4 zeroed device words the kernel writes
 * only if a bounded wait gives up (read them with fk_status_check).
 */
int fk_gemm_bf16_launch(const void* a_map, const void* b_map, const void* c_map, uint32_t m,
                        uint32_t n, uint32_t k, uint32_t group, void* stream,
                        uint32_t* device_status);

/* Convenience over the three map builders + the launch, from device pointers
 * (what `gemm::run` does between staging and read-back, :506-536). */
int fk_gemm_bf16(const void* a, const void* b, void* c, uint32_t m, uint32_t n, uint32_t k,
                 uint32_t ldc, uint32_t group, void* stream, uint32_t* device_status);

/* The same kernel behind two switches, for the callers next to the path:
 *   FK_GEMM_F16_OPERANDS  A and B are fp16 (maps built with FK_F16), C stays bf16: the operand
 *                         types of `gemm_sol` (examples/src/gemm_sol.rs:6-8, 202-207), whose
 *                         [512, 256] cluster tile is this kernel's own.
 *   FK_GEMM_ACCUMULATE    C += A.B^T: the epilogue's stores become the copy engine's
 *                         reduce-add (`tma_store_add_2d`, src/shared.rs:974-1009;
 *                         `commit_add_2d`, src/epilogue.rs:789-812): the rounded bf16 tile is
 *                         added into C in bf16, C is never read by a thread, and C must hold
 *                         values beforehand.
 *   FK_GEMM_RELU          max(x, 0) on the fp32 value before its one rounding to bf16: the `Relu`
 *                         unary map on a register tile (src/reg.rs:261, 1502-1504).
 *   FK_GEMM_TILE_NARROW / FK_GEMM_TILE_WIDE  pick the kernel instead of letting the launch choose:
 *                         the wide one (persistent two-CTA clusters, [512, 256] items) or the
 *                         narrow one (one CTA per [128, 128] tile, two CTAs an SM), which the
 *                         reference ships as its own entry for launches at or below half a wave
 *                         (`gemm_sol_m256_n128`, examples/src/gemm_sol.rs:1063, dispatch :1335-1337).
 *                         Unasked, a launch of at most 128 narrow tiles, or of at most two per SM
 *                         with K <= 2048, takes the narrow tile; with K >= 4096 and SMs to spare
 *                         a tile's k-blocks are cut across a cluster of two or four CTAs that
 *                         hand their fp32 tiles to the first through distributed shared memory.
 *                         Same operand maps, same C map, same results up to fp32 summation order.
 *   FK_GEMM_ORDER_FEED / FK_GEMM_ORDER_STATIC  pick how the wide kernel's clusters get their items
 *                         instead of letting the launch choose (the reference's two item loops,
 *                         `run_stealing` and `run`, src/pipeline.rs:613-660, 226-273): one cluster per item in the grid,
 *                         the resident clusters taking the others' items over through cluster
 *                         launch control (the items in flight are then always the next ones of the
 *                         traversal), or cluster c walking items c, c + clusters, ... . Unasked, a
 *                         launch of at least four waves of items of at least 32 k-blocks is fed.
 *                         Same results either way.
 * The `_fused` entries also take `bias`: null, or n bf16 values (16-byte aligned) added per column
 * in fp32 before the rounding -- a column vector every row shares (`load_vec` / `add_col`,
 * src/global.rs:410-416, as examples/src/layernorm.rs:200-203 uses them for beta). Bias first,
 * then the map, then (with FK_GEMM_ACCUMULATE) the add into C.
 * fk_gemm_bf16_launch / fk_gemm_bf16 are these with flags = 0 and no bias. */
/* The traversal width (`group`, the reference's x8, examples/src/gemm.rs:138) this kernel measures
 * best with on a 148-SM part: its 74 items in flight then cover 6 x 12.3 tiles, the fewest operand
 * panel bytes per wave for [512, 256] items. */
#define FK_GEMM_GROUP 6u
/* The same for a given shape and device: FK_GEMM_GROUP's rule, sqrt(clusters / 2), and two thirds of it
 * for a matrix with fewer tile columns than the items in flight span (an eighth of 16384 columns). */
uint32_t fk_gemm_group(uint32_t m, uint32_t n, uint32_t sm_count);
#define FK_GEMM_F16_OPERANDS 1u
#define FK_GEMM_ACCUMULATE 2u
#define FK_GEMM_RELU 4u
#define FK_GEMM_TILE_NARROW 8u
#define FK_GEMM_TILE_WIDE 16u
#define FK_GEMM_ORDER_FEED 32u
#define FK_GEMM_ORDER_STATIC 64u
int fk_gemm_launch_fused(const void* a_map, const void* b_map, const void* c_map, const void* bias, uint32_t m,
                         uint32_t n, uint32_t k, uint32_t group, uint32_t flags, void* stream,
                         uint32_t* device_status);
int fk_gemm_fused(const void* a, const void* b, void* c, const void* bias, uint32_t m, uint32_t n, uint32_t k,
                  uint32_t ldc, uint32_t group, uint32_t flags, void* stream, uint32_t* device_status);
/* Items narrower than 256 columns. The persistent kernel's time is whole waves of items, so a launch
 * whose [512, 256] tile count sits just past a whole number of waves wastes most of its last wave:
 * 8192 x 3584 (an eighth of the 28672-column up-projection) is 3 waves of 74 and 2 tiles. Items of
 * 224 or 192 columns (the MMAs' N) can fill the waves better: 256 items of [512, 224] run in 3.06
 * wave-times of the wide item instead of 3.5. The entries that take pointers choose by themselves.
 * A caller that keeps its own maps (as the reference's `run` does, examples/src/gemm.rs:506-513) asks
 * fk_gemm_item_columns for the width this device would choose (256, 224 or 192) and builds B's map
 * with a box of item_columns / 2 rows, and for 224 a second store map of C with a [32, 32] box and
 * no swizzle (`c_tail_map`: the item's last 32 columns; null otherwise); fk_gemm_launch_tiled is
 * fk_gemm_launch_fused for such maps. */
uint32_t fk_gemm_item_columns(uint32_t m, uint32_t n, uint32_t k, uint32_t flags, uint32_t sm_count);
int fk_gemm_launch_tiled(const void* a_map, const void* b_map, const void* c_map, const void* c_tail_map,
                         uint32_t item_columns, const void* bias, uint32_t m, uint32_t n, uint32_t k,
                         uint32_t group, uint32_t flags, void* stream, uint32_t* device_status);
int fk_gemm_launch(const void* a_map, const void* b_map, const void* c_map, uint32_t m, uint32_t n,
                   uint32_t k, uint32_t group, uint32_t flags, void* stream, uint32_t* device_status);
int fk_gemm(const void* a, const void* b, void* c, uint32_t m, uint32_t n, uint32_t k, uint32_t ldc,
            uint32_t group, uint32_t flags, void* stream, uint32_t* device_status);

/* Launches under one wave. The reference switches to a narrow `[256, 128]` cluster tile when a
 * launch holds at most half a wave of its wide tiles (`gemm_sol_m256_n128`,
 * examples/src/gemm_sol.rs:1063, dispatch :1335-1337), so that more SMs take part; this entry
 * reaches the idle SMs by splitting K instead: every item's k-blocks are cut into runs, one per
 * cluster, each run adds its fp32 tile into `workspace` through the copy engine's reduce-add
 * (`tma_store_add_2d`, src/shared.rs:974-1009, on fp32 here: the sums are rounded to bf16 ONCE,
 * after the last run, by whichever run arrives last), bias / ReLU / accumulate as in fk_gemm_fused.
 *   fk_gemm_workspace_bytes: bytes the shape needs on a device of `sm_count` SMs, 0 when it
 *     would not be split: the runs' fp32 tiles cross the L2 twice, and the narrow tile with K cut
 *     across a cluster of CTAs (every GEMM entry does that by itself) is faster wherever a launch
 *     has tiles enough, so this path takes launches of at most 16 narrow tiles with K >= 32768;
 *   `workspace`: device memory, 16-byte aligned, ALL ZERO before its first use -- every launch
 *     leaves it all zero again, so it is cleared once, not per call. Launches that share a
 *     workspace must not overlap on the device. With a null workspace, or a shape that would not
 *     be split, the call is fk_gemm_fused. */
uint64_t fk_gemm_workspace_bytes(uint32_t m, uint32_t n, uint32_t k, uint32_t sm_count);
int fk_gemm_fused_workspace(const void* a, const void* b, void* c, const void* bias, uint32_t m, uint32_t n,
                            uint32_t k, uint32_t ldc, uint32_t group, uint32_t flags, void* workspace,
                            uint64_t workspace_bytes, void* stream, uint32_t* device_status);

/* The whole of `gemm::run` from HOST buffers (:503-537): stage A and B, launch,
 * read C back; blocks until C is on the host. Device buffers are cached per
 * device and grown on demand. One call at a time per device: the staging buffers, the three
 * streams and the status words belong to the device, so the call holds a per-device lock from
 * its first enqueue to its last wait and a second thread calling on the same device waits its
 * turn (fk_flash_fwd_host and fk_gemm_bf16_host_noalloc take the same lock). Every wait inside
 * carries the launch deadline (fk_launch_budget_ms) and the call leaves none of its copies in
 * flight behind any return, error returns included. */
int fk_gemm_bf16_host(const uint16_t* a_host, const uint16_t* b_host, uint16_t* c_host, uint32_t m,
                      uint32_t n, uint32_t k, uint32_t group);

/* No counterpart in the reference. fk_gemm_bf16_host for callers that must not reach the CUDA
 * allocator from this call (a latency-bound serving loop that cannot take the device-wide
 * synchronisation of cudaMalloc/cudaFree; a process whose device memory is already handed out
 * in full to another pool): A, B, C and the status words are staged in an array that is part of
 * the library image, so the call allocates nothing. Limits and rules:
 *   - each of A (m*k), B (n*k) and C (m*n) at most 8 MiB of bf16; larger shapes are refused
 *     with FK_ERR_TOO_LARGE and a message naming the sizes;
 *   - every GPU that loads the library holds the 24 MiB + 256 B array until the process exits;
 *   - the first call on a device looks the array's device address up (cudaGetSymbolAddress);
 *     make that first call outside any stream capture;
 *   - all calls on a device share the array, which keeps the previous call's contents (the
 *     call clears what must start at zero): two calls that overlap on the GPU race. The call
 *     itself runs on the default stream and returns once C is on the host. */
int fk_gemm_bf16_host_noalloc(const uint16_t* a_host, const uint16_t* b_host, uint16_t* c_host,
                              uint32_t m, uint32_t n, uint32_t k, uint32_t group);

/* Flash-attention forward: `kernels::flash_forward` + `flash_forward::run`'s
 * guards (examples/src/flash_forward.rs:151-158, 477-483), widened to a batch,
 * a non-causal mode, bf16 output and a log-sum-exp vector. Q, K, V and O are
 * packed [planes = batch*heads, seq, 128] bf16; lse is [planes, seq] fp32
 * (natural log), may be null. Like the reference kernel's `out`, the output is a
 * device pointer the kernel stores rows through: `o_bf16` ([planes, seq, 128]
 * bf16, 16-byte aligned), or, when `o_f32` is non-null, fp32 [planes, seq, 128]
 * (the reference kernel's own output type) instead.
 *   q_map / k_map / v_map: fk_encode_bf16_panels(base, 128 box rows, 128, seq, planes)
 * Requires seq % 128 == 0, planes >= 1. One persistent CTA per SM walks the
 * (query block, plane) items. `device_status` as for the GEMM. */
int fk_flash_fwd_launch(const void* q_map, const void* k_map, const void* v_map, void* o_bf16,
                        float* o_f32, float* lse, uint32_t planes, uint32_t seq, float scale,
                        int causal, void* stream, uint32_t* device_status);

/* Convenience from device pointers. */
int fk_flash_fwd(const void* q, const void* k, const void* v, void* o_bf16, float* o_f32,
                 float* lse, uint32_t planes, uint32_t seq, float scale, int causal, void* stream,
                 uint32_t* device_status);

/* From HOST buffers: stage Q, K, V, launch, read O (bf16) and lse back. */
int fk_flash_fwd_host(const uint16_t* q_host, const uint16_t* k_host, const uint16_t* v_host,
                      uint16_t* o_host, float* lse_host, uint32_t planes, uint32_t seq, float scale,
                      int causal);

/* Flash-attention backward, D = 128: dQ, dK, dV from Q, K, V, O, dO and the log-sum-exp the
 * forward wrote (natural log, [planes, seq] fp32). The reference has no backward kernel; it
 * carries its pieces (`mma_atb` / `mma_atbt`, src/mma.rs:314-376; `make_causal_t_at`,
 * src/reg.rs:1432-1434; LSE vector loads, src/global.rs:573-654) and names it the next caller of
 * the forward's LSE. All tensors packed [planes, seq, 128] bf16; seq % 128 == 0. `workspace` is
 * fk_flash_bwd_workspace_bytes(planes, seq) bytes of device memory, 16-byte aligned, written by
 * the call (per-row statistics); nothing is allocated. Three launches on `stream`, no atomics:
 * results do not depend on scheduling. `device_status` as for the GEMM. */
uint32_t fk_flash_bwd_shared_bytes(void);
uint32_t fk_flash_bwd_threads(void);
uint64_t fk_flash_bwd_workspace_bytes(uint32_t planes, uint32_t seq);
int fk_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                 const float* lse, void* dq, void* dk, void* dv, float* workspace, uint32_t planes,
                 uint32_t seq, float scale, int causal, void* stream, uint32_t* device_status);

/* ---------------------------------------------------------------- row kernels
 *
 * The memory-bound kernels either side of attention and GEMM, over rows of 128 bf16 columns
 * (row-major, packed; 16-byte aligned buffers; `destination` may equal `source`). The
 * reference launches them with tensor maps over [128, 128] tiles; these entries take the
 * buffers themselves because a tile of whole rows is contiguous and moves by bulk copy.
 * `device_status` as for the GEMM. Asynchronous on `stream`.
 *
 * fk_softmax_rows:   `kernels::softmax_rows` (examples/src/softmax.rs:176-186, run :215-300):
 *                    y = 2^(x - max(x)) / sum, per row of [planes, rows_per_plane, 128];
 *                    rows_per_plane % 128 == 0.
 * fk_layernorm_rows: `kernels::layernorm_rows` (examples/src/layernorm.rs:140-214):
 *                    y = gamma * (x - mean) / sqrt(var + epsilon) + beta per row of [rows, 128];
 *                    gamma, beta [128] bf16; rows % 128 == 0.
 * fk_groupnorm_tile: `kernels::groupnorm_tile` (examples/src/layernorm.rs:232-306):
 *                    y = (x - mean) / sqrt(var + epsilon) with the statistics of each
 *                    [128, 128] tile of [rows, 128]; rows % 128 == 0. */
uint32_t fk_rows_shared_bytes(void);
uint32_t fk_rows_threads(void);
int fk_softmax_rows(const void* source, void* destination, uint32_t rows_per_plane, uint32_t planes,
                    void* stream, uint32_t* device_status);
int fk_layernorm_rows(const void* source, const void* gamma, const void* beta, void* destination,
                      uint32_t rows, float epsilon, void* stream, uint32_t* device_status);
int fk_groupnorm_tile(const void* source, void* destination, uint32_t rows, float epsilon,
                      void* stream, uint32_t* device_status);

/* ---------------------------------------------------------------- waits and status
 *
 * `watchdog::wait` / `wait_event` (src/watchdog.rs:300-332): poll with a
 * deadline instead of blocking in a synchronize: spin for the first 50 ms, then one poll per
 * millisecond (`SPIN`, `POLL`, :117-121). Unlike the reference these return FK_ERR_TIMEOUT
 * rather than aborting the process. */
int fk_wait_stream(void* stream, uint32_t budget_ms);
int fk_wait_event(void* event, uint32_t budget_ms);

/* `watchdog::budget` (src/watchdog.rs:102-106): the deadline of every wait the library makes on
 * its own (fk_status_check and the host-buffer entry points): 30 000 ms unless the
 * environment variable KITTENS_LAUNCH_BUDGET_MS holds another value. Read once per process. */
uint32_t fk_launch_budget_ms(void);

/* Self-tests of the host-side waiting, no device needed. fk_selftest_deadline runs the poll loop
 * of fk_wait_stream against a query that answers "not ready" `ready_after_polls` times
 * (0xffffffff: for ever) and then "done": FK_OK, or FK_ERR_TIMEOUT after `budget_ms`.
 * fk_selftest_call_guard takes the per-device lock of the host-buffer entry points, holds it
 * for `hold_ms` and reports when it got and gave up the lock (steady-clock nanoseconds): two
 * threads calling it for one device must not overlap. */
int fk_selftest_deadline(uint32_t budget_ms, uint32_t ready_after_polls);
int fk_selftest_call_guard(int device, uint32_t hold_ms, uint64_t* entered_ns, uint64_t* left_ns);

/* Read a kernel's 4 status words back (waiting on `stream` under the launch
 * deadline) and, when the first is non-zero, return FK_ERR_DEVICE_STALL with the role, block, stage and
 * parity in fk_last_error(). */
int fk_status_check(const uint32_t* device_status, void* stream);

/* `Semaphore::wait_before(parity, ticks)` giving up (src/sync.rs:214-245), as a self-test: launches
 * one warp that waits `budget_cycles` on a barrier nothing arrives on, records the expiry in the 4
 * zeroed `device_status` words and exits normally. fk_status_check then reports
 * FK_ERR_DEVICE_STALL; the context stays usable. */
int fk_selftest_stall(void* stream, uint32_t* device_status, uint32_t budget_cycles);

/* `exp2_approx` (src/reg.rs:81-93) as the attention kernels compute it for a share of their
 * exponentials (the same split and polynomial, on packed fp32 pairs with fused multiply-adds):
 * y[i] = 2^x[i] for `count` (even) device floats, so that a test can hold the device arithmetic to
 * the bound the reference's own test states (relative error under 1e-4 over [-125, 125],
 * src/reg.rs:2047-2062). */
int fk_selftest_exp2(const float* x, float* y, uint32_t count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FERRO_KITTENS_H */
