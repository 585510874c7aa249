// tcgen05 / TMA / mbarrier PTX wrappers shared by the tensor-core BitLinear kernels (sm_100a).
#pragma once
#include <cuda.h>

#include "bitlinear.cuh"

namespace {

constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;   // bounded device-side waits: about one second of SM clock

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait (about one second of SM clock): returns false, with *abort_flag set, if the phase never
// completes or another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    // try_wait suspends the thread in hardware for a while; the clock and the abort flag are only looked at
    // now and then so that waiting warps do not compete with the MMA-issuing thread for issue slots
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            return false;
        }
    }
}

// Wait of a role that is not on the critical path (a producer ahead of its consumers, unpack warps with a full
// ring): polls with a short sleep in between so that it does not take issue slots from the warps that are.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 4; ++i)
        if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            if (mbar_try(bar, parity)) return true;
            __nanosleep(40);
        }
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            return false;
        }
    }
}
// Whole-warp wait: lane 0 polls (with or without sleeping between polls), then every lane observes the completed phase itself (its own acquire).
template <bool RELAXED>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0)
        ok = (RELAXED ? mbar_wait_relaxed(bar, parity, abort_flag) : mbar_wait(bar, parity, abort_flag)) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok) {
        int tries = 0;
        while (!mbar_try(bar, parity) && ++tries < 100000) {}
        ok = __all_sync(0xffffffffu, tries < 100000) ? 1 : 0;
        if (!ok) *abort_flag = 1;
    }
    return ok != 0;
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t.reg .b32 r;\n\t"
        "elect.sync r|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Fetch a tensor map into the descriptor cache ahead of its first use: the first TMA copy of a kernel otherwise pays
// for the 128-byte descriptor read from the kernel's parameter space on its critical path (after the grid-dependency wait)
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// shared memory -> global memory (tiled TMA store); completion is tracked per thread in bulk groups
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the newest N bulk groups of this thread have finished READING their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make generic-proxy writes to shared memory visible to the async proxy (TMA)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], int8 x int8 -> int32
__device__ __forceinline__ void mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(addr)
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- forms for a pair of CTAs working as one MMA unit (cta_group::2): one thread of the even CTA of the pair issues
// MMAs of 256 rows (128 of A and of D in each CTA's tensor memory) whose B operand is split between the two CTAs'
// shared memories.  Every tcgen05 instruction of such a kernel that takes a cta_group carries ::2.
template <int CG> __device__ __forceinline__ void tmem_alloc_cg(uint32_t* slot, uint32_t cols) {
    if constexpr (CG == 2) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
        tmem_alloc(slot, cols);
    }
}
template <int CG> __device__ __forceinline__ void tmem_dealloc_cg(uint32_t addr, uint32_t cols) {
    if constexpr (CG == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
    else tmem_dealloc(addr, cols);
}
// commit of the pair's MMAs: arrives on the barrier at this offset in both CTAs of the pair (CG == 2) or in this CTA
template <int CG> __device__ __forceinline__ void tc_commit_cg(uint64_t* bar) {
    if constexpr (CG == 2)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
    else tc_commit(bar);
}
template <int CG> __device__ __forceinline__ void mma_i8_ts_cg(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (CG == 2)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else mma_i8_ts(d_tmem, a_tmem, b_desc, idesc, accumulate);
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the object at `my_smem_addr` in the CTA with rank `rank` of this cluster
__device__ __forceinline__ uint32_t cluster_addr(const void* my_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(my_smem_addr)), "r"(rank));
    return r;
}
// Arrive on a barrier of another CTA of the cluster.  Relaxed: what the arrival announces (tensor-memory stores that
// tcgen05.wait::st has seen complete, accumulator columns already read into registers) is finished before the
// instruction issues, and a release at cluster scope stalls the arriving thread for most of a microsecond.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// tiled load into this CTA's shared memory whose completion bytes are credited to a barrier of the pair's other CTA
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t cluster_bar_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(cluster_bar_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Phase trace for kernel experiments, compiled only into the experiments build (-DMMF_EXPERIMENTS): CTA (0,0,0) writes
// clock64 stamps into the workspace header when word 1 of the workspace holds MMF_TRACE_MAGIC.  In the product build
// MMF_TRACE_PTR(...) is a null constant and every trace statement folds away (no extra load in any kernel prologue).
#ifdef MMF_EXPERIMENTS
constexpr int MMF_TRACE_MAGIC = 0x7ace;
#define MMF_TRACE_PTR(...) (__VA_ARGS__)
__device__ __forceinline__ long long trace_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));   // nanoseconds, comparable across SMs and launches
    return t;
}
__device__ __forceinline__ void trace_mark(long long* trace, int slot) {
    if (trace) trace[slot] = trace_now();
}
// one record of 32 stamps per traced launch: word 2 of the workspace counts launches, records start at word 16
__device__ __forceinline__ long long* trace_record(int32_t* ws) {
    const int idx = atomicAdd(ws + 2, 1);
    return idx < 2000 ? reinterpret_cast<long long*>(ws + 16) + 32 * idx : nullptr;
}
#else
#define MMF_TRACE_PTR(...) (static_cast<long long*>(nullptr))
__device__ __forceinline__ void trace_mark(long long*, int) {}
__device__ __forceinline__ long long trace_now() { return 0; }   // only reached behind a null trace pointer
#endif

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
    d |= (uint64_t)1 << 16;                          // leading-dim byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride-dim byte offset: next 8-row group
    d |= (uint64_t)1 << 46;                          // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
    return d;
}

}  // namespace
