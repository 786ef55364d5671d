// Shared device-side building blocks for the sm_100a kernels: mbarrier and TMA
// wrappers, tcgen05 (UMMA / tensor memory) wrappers, descriptor encoders and the
// bounded-wait + status-word protocol.
//
// Every wait on an mbarrier in this library goes through mbar_wait_bounded():
// it gives up after a fixed number of polls, records where it gave up in a
// global status word and raises a CTA-wide abort flag, so a protocol bug shows
// up as KAIO_B200_ERR_TIMEOUT on the host instead of a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kaio {

// ---------------------------------------------------------------- status word
// Layout of the per-device status block (uint32_t[4]) in global memory:
//   [0] first error code (0 = none), [1] blockIdx.x of the reporter,
//   [2] site id inside the kernel,   [3] kernel id.
enum : uint32_t {
    DEV_OK = 0,
    DEV_TIMEOUT = 1,
    DEV_BAD_LAYOUT = 2,  // a kernel found its shared-memory window laid out unexpectedly
};

enum : uint32_t {
    KERNEL_W8A8 = 1,
    KERNEL_W4A16_DECODE = 2,
    KERNEL_DQ_GEMM = 3,
    KERNEL_FLASH_ATTN = 4,
    KERNEL_SELFTEST = 5,
};

__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code, uint32_t site,
                                              uint32_t kernel_id)
{
    if (status != nullptr && atomicCAS(status, 0u, code) == 0u) {
        status[1] = blockIdx.x;
        status[2] = site;
        status[3] = kernel_id;
        __threadfence();
    }
}

// ---------------------------------------------------------------- addresses
__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "elect.sync _|P, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait with a suspend-time hint: the hardware parks the thread until the phase completes
// or `hint_ns` elapse, so a waiting warp does not compete for issue slots with the warps that
// do the work (a spinning waiter on the same scheduler slows a single-thread MMA issuer or TMA
// producer several-fold).
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Each poll may park for up to WAIT_HINT_NS; WAIT_POLL_LIMIT polls bound a wait to about one
// second (the hint is an upper bound, so the limit also counts polls that return early).
#ifndef KAIO_WAIT_HINT_NS
#define KAIO_WAIT_HINT_NS 20000
#endif
constexpr uint32_t WAIT_HINT_NS = KAIO_WAIT_HINT_NS;
constexpr uint32_t WAIT_POLL_LIMIT = 1u << 20;

// ~1 s at 2 GHz: the bound of every wait in the shipped kernels.
constexpr unsigned long long WAIT_CYCLE_LIMIT = 2000000000ull;

// One lane's wait with an explicit cycle budget.  Returns true when the phase completed; false
// when this wait (or another thread of the CTA, through *abort_flag) gave up.  Giving up raises
// the abort flag, records {DEV_TIMEOUT, block, site, kernel} in the status block and returns:
// no trap, the kernel runs to its normal end.
__device__ __forceinline__ bool mbar_wait_lane_budget(uint32_t bar, uint32_t parity,
                                                      volatile uint32_t* abort_flag,
                                                      uint32_t* status, uint32_t site,
                                                      uint32_t kernel_id,
                                                      unsigned long long max_cycles)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const unsigned long long t_start = clock64();
    for (uint32_t it = 0; it < WAIT_POLL_LIMIT; ++it) {
        if (mbar_try_wait_hint(bar, parity, WAIT_HINT_NS))
            return true;
        if (*abort_flag)
            return false;
        // polls that return early (hint not honoured) must not shorten or lengthen the bound
        // by orders of magnitude
        if (clock64() - t_start > max_cycles)
            break;
    }
    *abort_flag = 1;
    report_status(status, DEV_TIMEOUT, site, kernel_id);
    return false;
}

// One lane's wait with the library's standard bound.
__device__ __forceinline__ bool mbar_wait_lane(uint32_t bar, uint32_t parity,
                                               volatile uint32_t* abort_flag, uint32_t* status,
                                               uint32_t site, uint32_t kernel_id)
{
    return mbar_wait_lane_budget(bar, parity, abort_flag, status, site, kernel_id,
                                 WAIT_CYCLE_LIMIT);
}

__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// WARP-COLLECTIVE polling wait for the few warps whose reaction time bounds a pipeline (a TMA
// producer, an MMA issuer): it polls with the non-blocking test_wait instead of parking in
// try_wait, so it sees the phase flip within tens of cycles.  Same bound and same give-up
// protocol as mbar_wait_bounded.  Only lane 0 polls; the outcome is broadcast.
__device__ __forceinline__ bool mbar_wait_polling(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag, uint32_t* status,
                                                  uint32_t site, uint32_t kernel_id)
{
    bool ok = true;
    if ((threadIdx.x & 31u) == 0) {
        ok = mbar_test_wait(bar, parity);
        if (!ok) {
            const unsigned long long t_start = clock64();
            for (;;) {
                if (mbar_test_wait(bar, parity)) {
                    ok = true;
                    break;
                }
                if (*abort_flag)
                    break;
                if (clock64() - t_start > WAIT_CYCLE_LIMIT) {
                    *abort_flag = 1;
                    report_status(status, DEV_TIMEOUT, site, kernel_id);
                    break;
                }
            }
        }
    }
    return __all_sync(0xffffffffu, ok);
}

// WARP-COLLECTIVE wait: all 32 lanes of a warp call it together.  Lanes can leave the polling
// loop at different times (one lane may have been busy arriving on another barrier), and the
// loop's give-up exit keeps the compiler from re-converging them right behind it; the closing
// vote does, and makes the outcome uniform.  The `.sync.aligned` tcgen05 instructions (ld, st,
// alloc) that follow a wait need exactly that: executed by a diverged warp their result is
// undefined (seen as a rare wrong value in the lane that had done the extra arrive).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag, uint32_t* status,
                                                  uint32_t site, uint32_t kernel_id)
{
    const bool ok = mbar_wait_lane(bar, parity, abort_flag, status, site, kernel_id);
    return __all_sync(0xffffffffu, ok);
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 2-D tiled load global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* tmap,
                                            uint32_t bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// Same with an L2 cache-policy hint (createpolicy result).
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* tmap,
                                                 uint32_t bar, int32_t x, int32_t y,
                                                 uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y),
        "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// 2-D tiled store shared -> global (bulk group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, uint32_t src_smem, int32_t x,
                                             int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src_smem), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_store_commit()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_all()
{
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- tensor memory
template <uint32_t NCOLS>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "n"(NCOLS)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

template <uint32_t NCOLS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(NCOLS)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Arrives (count 1) on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     bar)
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], s8 x s8 -> s32.
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], f16 x f16 -> f32.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane
// (lane-quarter base + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Shared-memory address of `addr` (an address in this CTA's window) inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}

// Arrive (count 1) on an mbarrier of another CTA of the cluster (address from mapa_shared).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar)
                 : "memory");
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One lane's wait on a local mbarrier whose arrivals may come from the peer CTA (cluster-scope
// acquire).
__device__ __forceinline__ bool mbar_wait_lane_cluster(uint32_t bar, uint32_t parity,
                                                       volatile uint32_t* abort_flag,
                                                       uint32_t* status, uint32_t site,
                                                       uint32_t kernel_id)
{
    const unsigned long long t_start = clock64();
    for (uint32_t it = 0; it < WAIT_POLL_LIMIT; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred P;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2, %3;\n"
            "selp.u32 %0, 1, 0, P;\n"
            "}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(WAIT_HINT_NS)
            : "memory");
        if (ok)
            return true;
        if (*abort_flag)
            return false;
        if (clock64() - t_start > WAIT_CYCLE_LIMIT)
            break;
    }
    *abort_flag = 1;
    report_status(status, DEV_TIMEOUT, site, kernel_id);
    return false;
}

// Warp-collective form (see mbar_wait_bounded).
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint32_t bar, uint32_t parity,
                                                          volatile uint32_t* abort_flag,
                                                          uint32_t* status, uint32_t site,
                                                          uint32_t kernel_id)
{
    const bool ok = mbar_wait_lane_cluster(bar, parity, abort_flag, status, site, kernel_id);
    return __all_sync(0xffffffffu, ok);
}

// 2-D tiled load global -> this CTA's shared memory whose completion bytes are credited to an
// mbarrier that may live in the peer CTA of the pair (`bar` is a cluster address from
// mapa_shared).  A plain, single-destination load.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* tmap,
                                                 uint32_t bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

template <uint32_t NCOLS>
__device__ __forceinline__ void tmem_alloc_2cta(uint32_t smem_dst)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "n"(NCOLS)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_2cta()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

template <uint32_t NCOLS>
__device__ __forceinline__ void tmem_dealloc_2cta(uint32_t taddr)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "n"(NCOLS)
                 : "memory");
}

// Pair MMA: D (256 rows: 128 in each CTA's tensor memory) (+)= A (128 rows from each CTA's shared
// memory) * B (N columns, half from each CTA's shared memory); issued by the leader CTA only.
__device__ __forceinline__ void umma_i8_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_f16_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives (count 1) on the mbarrier at the same shared-memory offset in every CTA of `cta_mask`
// once all pair MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar, uint16_t cta_mask)
{
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   bits [0,14)  start address >> 4        bits [16,30) leading-dim byte offset >> 4
//   bits [32,46) stride-dim byte offset >> 4   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) swizzle mode (2 = 128-byte)
// K-major operand (rows of 128 bytes along K): stride offset = distance between
// 8-row groups (1024 B for a dense tile), leading offset unused.
// MN-major operand (rows of 128 bytes along M/N, one row per k): stride offset =
// distance between 8-k groups, leading offset = distance between 128-byte chunks
// along M/N.
__host__ __device__ constexpr uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes)
{
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}

// The same descriptor with the 64-byte swizzle mode (operand rows of 64 bytes; 8-row groups are
// then 512 bytes apart in a dense tile).
__host__ __device__ constexpr uint64_t make_smem_desc_sw64(uint32_t smem_addr, uint32_t lbo_bytes,
                                                           uint32_t sbo_bytes)
{
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)4 << 61);
}

// Instruction descriptor for kind::i8 / kind::f16 (dense, no negate, no saturate).
//   bits [4,6) D format (1 = f32, 2 = s32)   bits [7,10) A format   bits [10,13) B format
//   bit 15 A major (0 = K, 1 = MN)           bit 16 B major
//   bits [17,23) N >> 3                      bits [24,29) M >> 4
// Formats: kind::f16: 0 = f16, 1 = bf16;  kind::i8: 0 = u8, 1 = s8.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t m, uint32_t n)
{
    return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
           ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Byte offset of logical (row, 16-byte chunk) inside a 128-byte-swizzled tile whose
// rows are 128 bytes and whose base is 1024-byte aligned (the pattern TMA writes and
// UMMA reads with the 128-byte swizzle mode).
__host__ __device__ constexpr uint32_t sw128_offset(uint32_t row, uint32_t chunk16)
{
    return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

}  // namespace kaio
