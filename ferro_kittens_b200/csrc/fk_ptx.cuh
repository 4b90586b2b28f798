// Inline-PTX wrappers for the sm_100a instructions the two kernels use:
// mbarrier semaphores, TMA tiled loads/stores, tcgen05 tensor memory, MMA,
// commit and fences, and the cluster rendezvous.
//
// Restates, as free functions, the subset of the reference's `sync` (src/sync.rs:123-312),
// `shared` TMA movers (src/shared.rs:644-1009), `tmem` (src/tmem.rs:112-224) and
// `mma` (src/mma.rs:137-146, 413-434, 543-565) modules that its two kernels reach.
// No TMA load here carries a cluster-multicast qualifier: a pair's two CTAs
// each fetch their own halves of both operands.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace fk {

// ---------------------------------------------------------------- addresses

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

/// shared::cluster address of `cta_addr` (a shared::cta address) in CTA `rank`.
__device__ __forceinline__ uint32_t mapa(uint32_t cta_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(cta_addr), "r"(rank));
    return out;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_count_x() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\t"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
/// 16 bytes into the shared memory of any CTA of the cluster (a shared::cluster address from `mapa`).
__device__ __forceinline__ void st_shared_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c,
                                                     uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c),
                 "r"(d)
                 : "memory");
}
/// Makes what peer CTAs wrote into this CTA's shared memory before their release-arrive visible
/// to the loads that follow a wait on the barrier they arrived on.
/// Bulk copy from this CTA's shared memory into a peer CTA's (both addresses and the size multiples
/// of 16 bytes), completing `bytes` on an mbarrier of the cluster (the peer's, as a rule). The
/// source may be reused once that barrier's phase has completed.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                  uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            dst_cluster_addr),
        "r"(src_cta_addr), "r"(bytes), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void fence_acq_rel_cluster() {
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
/// Makes freshly initialised barriers visible to the async proxy and to the peer CTA.
__device__ __forceinline__ void fence_mbarrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
/// Generic-proxy writes to shared memory before, async-proxy (TMA / MMA) reads after.
__device__ __forceinline__ void fence_proxy_async_shared() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
/// Orders this thread's async-proxy accesses to global memory (bulk copies and reductions) with
/// its generic-proxy accesses to the same addresses.
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
/// Arrive on a barrier named by a shared::cluster address (own or peer CTA).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
                 : "memory");
}
// How long one try_wait may keep the thread suspended in hardware (ns). The
// thread wakes as soon as the phase completes, so a long hint costs no latency;
// it only keeps waiting roles from spending issue slots on polling.
constexpr uint32_t kSuspendHintNs = 200000;

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}

// Where a bounded wait gave up: written once per launch into the caller's
// status words {code, block, detail, parity}. 0 means the launch ran clean.
// Cycle budget of one wait. About a second at the clocks a B200 runs at; the
// longest legitimate wait in either kernel is one tile's main loop (tens of
// microseconds).
constexpr long long kWaitBudgetCycles = 1ll << 31;

struct StallSite {
    uint32_t* status;        // global, may be null
    volatile uint32_t* stop; // shared: raised once any role gives up
    uint32_t peer_stop;      // shared::cluster address of the peer's flag, 0 if none
    long long budget = kWaitBudgetCycles;
    bool spin = false;       // poll with test_wait instead of suspending in try_wait
};

/// The non-suspending probe. A thread suspended in try_wait takes a few hundred cycles to come back
/// after the phase completes; a role on a kernel's critical path polls with this instead, at the
/// price of the issue slots the polling takes (so not for roles that wait most of the time).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

/// Parity wait with a deadline. Returns false when the budget ran out or
/// another role already raised `stop`; the caller must then fall through to
/// its teardown without issuing further asynchronous work. Follows the
/// reference's `Semaphore::wait_before` (src/sync.rs:214-245) and the shared
/// stop flag of its watched builds.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const StallSite& site,
                                          uint32_t code, uint32_t detail) {
    if (site.spin ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            if (site.spin ? mbar_test_wait(bar, parity) : mbar_try_wait(bar, parity)) return true;
        }
        if (*site.stop) return false;
        if (clock64() - start > site.budget) {
            *site.stop = 1;
            if (site.peer_stop) st_shared_cluster_u32(site.peer_stop, 1);
            if (site.status && atomicCAS(site.status, 0u, code) == 0u) {
                site.status[1] = blockIdx.x + gridDim.x * blockIdx.y;
                site.status[2] = detail;
                site.status[3] = parity;
            }
            return false;
        }
    }
}

// ---------------------------------------------------------------- TMA

/// One 2-D box into this CTA's shared memory, completing on `cluster_bar`,
/// which may live in either CTA of the pair (the leader's, in the GEMM).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0,
                                                 int c1, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     map),
                 "r"(src), "r"(c0), "r"(c1)
                 : "memory");
}
/// As `tma_store_2d`, but each element is ADDED into its destination, in the tensor map's own
/// element type, by the copy engine (reference: `tma_store_add_2d`, src/shared.rs:974-1009).
/// Same bulk-group completion as a plain store.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
        "r"(src), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1,
                                             int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
        "r"(src), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
/// At most `N` of this thread's store groups may still be reading shared memory.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
/// All of this thread's store groups have been written out.
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
/// Before a CTA exits: every store group has finished READING shared memory, which is all the CTA
/// still owes them; the writes themselves complete with the grid, like any other store in flight.
__device__ __forceinline__ void tma_store_wait_before_exit() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------- tcgen05: tensor memory

template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t columns) {
    if constexpr (CTA_GROUP == 2)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                     "r"(columns)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot),
                     "r"(columns)
                     : "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CTA_GROUP == 2)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    if constexpr (CTA_GROUP == 2)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address),
                     "r"(columns)
                     : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address),
                     "r"(columns)
                     : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

/// 32 lanes x 32 columns of fp32: lane i of the warp receives row
/// (address.lane + i), columns address.column .. +31, in v[0..31].
__device__ __forceinline__ void tmem_ld_32x32(uint32_t address, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
          "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(address)
        : "memory");
}
/// As `tmem_ld_32x32`, 8 columns wide.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t address, uint32_t (&v)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
        : "r"(address)
        : "memory");
}
/// As `tmem_ld_32x32`, 16 columns wide.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t address, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
          "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
          "=r"(v[14]), "=r"(v[15])
        : "r"(address)
        : "memory");
}
/// The store twin of `tmem_ld_32x32`, 16 columns wide.
__device__ __forceinline__ void tmem_st_32x16(uint32_t address, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(address),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t address, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
            address),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
        "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
        "r"(v[30]), "r"(v[31])
        : "memory");
}

// ---------------------------------------------------------------- tcgen05: MMA

/// D[tmem] (+)= A[smem] . B[smem], bf16 in, fp32 accumulate, K = 16 per issue.
template <int CTA_GROUP>
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    if constexpr (CTA_GROUP == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}
/// As `mma_ss` with the A operand read from tensor memory (bf16 pairs packed
/// in 32-bit columns, one row per lane).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

/// Cluster launch control (sm_100): a running cluster asks the hardware for the work of a cluster of
/// its grid that has not started yet. The 16-byte answer is written to shared memory at `response`
/// and completes 16 bytes on the mbarrier `bar`; a granted request means that cluster will never
/// start and its work is the asker's. After a refusal (nothing is left to take) no further request
/// may be made.
__device__ __forceinline__ void clc_try_cancel(uint32_t response, uint32_t bar) {
    asm volatile(
        "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];" ::"r"(response),
        "r"(bar)
        : "memory");
}
/// Decode the answer at `response`: true and the x index of the taken cluster's first CTA, or false.
__device__ __forceinline__ bool clc_query(uint32_t response, uint32_t& first_cta_x) {
    uint32_t granted, x = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b128 answer;\n\tld.shared.b128 answer, [%2];\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, answer;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, answer;\n\t}"
        : "=r"(granted), "+r"(x)
        : "r"(response)
        : "memory");
    first_cta_x = x;
    return granted != 0;
}

/// 1 in exactly one lane of a converged warp, 0 in the others. Use it as a BRANCH around the
/// whole issuing role (`if (elect_one()) { waits, MMAs, commits }`): the compiler then knows the
/// region runs in a single thread and emits the tight issue sequence -- 23 cycles of the thread's
/// own instructions per tcgen05.mma, measured, against 71 under `if (lane == 0)`, which it cannot
/// tell from arbitrary divergence. The waits, the MMAs and their commits must all sit inside the
/// one branch: tcgen05.commit tracks the MMAs issued by the thread that executes it, so a commit
/// executed by any other lane arrives at once, before the MMAs it was meant to cover have retired.
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t flag;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(flag));
    return flag;
}

/// Arrive on `cluster_bar` once every MMA this thread issued so far has retired.
template <int CTA_GROUP>
__device__ __forceinline__ void mma_commit(uint32_t cluster_bar) {
    if constexpr (CTA_GROUP == 2)
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                cluster_bar)
            : "memory");
    else
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                cluster_bar)
            : "memory");
}

// Register rebalancing between warpgroups (four consecutive warps, all of which must execute
// the same instruction): a warpgroup that only issues copies or MMAs gives registers back and a
// warpgroup that does arithmetic takes them. `inc` waits until the pool has them.
template <uint32_t REGISTERS>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}
template <uint32_t REGISTERS>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGISTERS));
}

// ---------------------------------------------------------------- misc

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t out;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
    return out;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
                 "r"(d)
                 : "memory");
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t (&v)[4]) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr)
                 : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 2^x for a pair, on the FMA pipe: clamp, split x = n + f with f in [-0.5, 0.5] by the
// 1.5 * 2^23 shift trick, a degree-3 minimax polynomial for 2^f (maximum relative error
// 7.5e-5, far inside a rounding to bf16), then n added into the exponent field. The same
// split the reference's `exp2_approx` makes (src/reg.rs:81-93), on packed fp32 pairs.
__device__ __forceinline__ float2 exp2_pair_fma(float2 x) {
    constexpr float kShift = 12582912.0f;  // 1.5 * 2^23
    x.x = fmaxf(x.x, -125.0f);
    x.y = fmaxf(x.y, -125.0f);
    const float2 shifted = __fadd2_rn(x, make_float2(kShift, kShift));
    const float2 whole = __fadd2_rn(shifted, make_float2(-kShift, -kShift));
    const float2 f = __ffma2_rn(whole, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(f, make_float2(0.05517166f, 0.05517166f), make_float2(0.24261113f, 0.24261113f));
    p = __ffma2_rn(p, f, make_float2(0.69326097f, 0.69326097f));
    p = __ffma2_rn(p, f, make_float2(0.99992806f, 0.99992806f));
    p.x = __int_as_float(__float_as_int(p.x) + (__float_as_int(shifted.x) << 23));
    p.y = __int_as_float(__float_as_int(p.y) + (__float_as_int(shifted.y) << 23));
    return p;
}
__device__ __forceinline__ float lg2_approx(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace fk
