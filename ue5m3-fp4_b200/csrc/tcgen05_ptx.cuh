// Inline-PTX wrappers for mbarrier, TMA, TMEM and tcgen05 on sm_100a, plus the bounded
// wait used by every kernel role.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ue5m3 {
namespace ptx {

constexpr long long kWaitBudgetClocks = 4000000000LL;  // about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Non-blocking probe of a phase: true when it has completed.  Used to look at the NEXT stage's
// barrier before issuing the current stage, so that the probe's latency overlaps the issue.
__device__ __forceinline__ bool mbar_test_wait(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// One lane of a converged warp.  Roles that issue TMA / tcgen05 instructions keep their
// control flow warp-uniform and predicate only the issue on this, so that addresses and
// descriptors stay in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xFFFFFFFF;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Bounded wait.  Returns false when the clock budget expired or another role raised the
// CTA's abort flag; on expiry records (site, iteration, block) in the caller's status words.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, uint32_t parity, int* abort_flag,
                                          int* status, int where, int iter) {
#pragma unroll 1
    for (int spin = 0; spin < 32; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 32; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*((volatile int*)abort_flag)) return false;
        if (clock64() - start > kWaitBudgetClocks) {
            *((volatile int*)abort_flag) = 1;
            if (status) {
                if (atomicCAS(&status[0], 0, 1) == 0) {
                    status[1] = where;
                    status[2] = iter;
                    status[3] = (int)blockIdx.x;
                }
            }
            return false;
        }
    }
}

// 2-D tiled TMA load into shared memory, completion counted on an mbarrier.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map,
                                            unsigned long long* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes,
                                          unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}

// mbarrier arrives once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
            smem_u32(bar))
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (no wait).
__device__ __forceinline__ void tmem_load_32_async(uint32_t taddr, uint32_t (&r)[32]) {
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

__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: 8-row groups 1024 bytes
// apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)1 << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    return desc;
}

// Shared-memory descriptor without swizzle for a [32 rows][16 bytes] block: core matrices
// of 8 rows x 16 bytes are 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_noswizzle_32x16(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)(128 >> 4) << 16;
    desc |= (uint64_t)(128 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    return desc;
}

// ---- CTA pairs (cluster of two, tcgen05 cta_group::2) ----------------------------------------

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}

// arrive on an mbarrier of any CTA of the cluster (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait_cluster(unsigned long long* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// mbar_wait with cluster-scope acquire, for barriers that the peer CTA (its threads, its TMA
// unit or the leader's commits) arrives on
__device__ __forceinline__ bool mbar_wait_cluster(unsigned long long* bar, uint32_t parity, int* abort_flag,
                                                  int* status, int where, int iter) {
    const long long start = clock64();
    while (true) {
#pragma unroll 1
        for (int spin = 0; spin < 32; ++spin)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*((volatile int*)abort_flag)) return false;
        if (clock64() - start > kWaitBudgetClocks) {
            *((volatile int*)abort_flag) = 1;
            if (status) {
                if (atomicCAS(&status[0], 0, 1) == 0) {
                    status[1] = where;
                    status[2] = iter;
                    status[3] = (int)blockIdx.x;
                }
            }
            return false;
        }
    }
}

// every thread of both CTAs of the cluster
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();  // the barrier instructions are warp-aligned: reconverge first
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// 2-D tiled TMA load into this CTA's shared memory whose completion is counted on an mbarrier
// given by shared::cluster address (the pair leader's); the data goes to this CTA only.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// arrives (on the mbarrier at a shared::cluster address) once every tcgen05 operation issued so
// far by this thread has completed in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
                 : "memory");
}

// round-half-even to an integer (torch.round), full-rate float ops only
__device__ __forceinline__ float rint_rne(float v) {
    float a = fabsf(v);
    float r = a < 8388608.0f ? __fadd_rn(__fadd_rn(a, 8388608.0f), -8388608.0f) : a;
    return copysignf(r, v);
}

}  // namespace ptx
}  // namespace ue5m3
