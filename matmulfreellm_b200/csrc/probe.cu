// Measurement aid: the int8 tensor-pipe peak of this GPU, measured with a bare tcgen05.mma kind::i8 issue
// loop (128 x 256 x 32 per instruction, A operand in tensor memory, B in shared memory, int32 accumulators
// in tensor memory), one CTA per SM.  Nothing is loaded or stored: operands are whatever the memories hold.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(128)
int8_mma_peak_kernel(int n_tokens, int iters, int* status, int commits, int issuers) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar[2];
    __shared__ __align__(8) uint64_t scratch_bar[2];   // target of the extra commits of the issue-cost experiment
    __shared__ uint32_t s_tmem;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // pseudo-random operand bytes: constant operands toggle few wires and let the GPU hold a clock that no real
    // contraction reaches under the power cap
    for (int i = threadIdx.x; i < (n_tokens * 128) / 4; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        reinterpret_cast<uint32_t*>(base)[i] = h;
    }
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[1])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&scratch_bar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&scratch_bar[1])) : "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    {   // A operand: 64 columns (8 K-steps of 32 bytes) of pseudo-random int8 for each of the 128 lanes
        const uint32_t lane_addr = (uint32_t)((threadIdx.x >> 5) * 32) << 16;
        for (int c = 0; c < 4; ++c) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                uint32_t h = (threadIdx.x * 64u + c * 16u + j) * 2654435761u + blockIdx.x * 7919u;
                h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
                r[j] = h;
            }
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                ::"r"(tmem + lane_addr + 256 + c * 16), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    // issue-cost experiment: with two issuers (n_tokens <= 128) the first thread of warps 0 and 1 each issue half of the
    // MMAs into an accumulator of their own — does the per-instruction issue cost of one thread overlap with the other's?
    const int who = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0 && who < issuers) {
        // shared-memory descriptor of a K-major, 128-byte-swizzled tile; instruction descriptor S32 += S8 x S8
        uint64_t bd = 0;
        bd |= (uint64_t)((smem_u32(base) & 0x3FFFFu) >> 4);
        bd |= (uint64_t)1 << 16;
        bd |= (uint64_t)(1024 >> 4) << 32;
        bd |= (uint64_t)1 << 46;
        bd |= (uint64_t)2 << 61;
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n_tokens >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint32_t acc = tmem + (uint32_t)who * 128u;
        const int mine = iters / issuers;
#pragma unroll 4
        for (int i = 0; i < mine; ++i) {
            const uint32_t a_addr = tmem + 256 + (uint32_t)(i & 7) * 8;
            const uint64_t b = bd + (uint64_t)((i & 3) * 2);
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                ::"r"(acc), "r"(a_addr), "l"(b), "r"(idesc), "r"(i > 0 ? 1u : 0u), "r"(0u)
                : "memory");
            // `commits` tcgen05.commit instructions after every fourth MMA, as a pipelined kernel issues them to release
            // its operand stages
            if ((i & 3) == 3)
                for (int c = 0; c < commits; ++c)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                                 ::"r"(smem_u32(&scratch_bar[c & 1])) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar[who])) : "memory");
        const long long t0 = clock64();
        uint32_t done = 0;
        while (!done) {   // bounded wait for the MMAs to retire
            asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\tselp.b32 %0, 1, 0, P1;\n\t}"
                         : "=r"(done) : "r"(smem_u32(&bar[who])), "r"(0u) : "memory");
            if (clock64() - t0 > 4000000000ll) { atomicExch(status, 1); break; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}


#ifdef MMF_EXPERIMENTS
// The same bare issue loop for a pair of CTAs (cluster of two, cta_group::2): the even CTA's thread 0 issues MMAs of
// 256 rows x n_tokens columns; each CTA holds 128 rows of A in tensor memory and n_tokens / 2 rows of B in shared memory.
// `commits`: a multicast tcgen05.commit after every fourth MMA.
__global__ void __launch_bounds__(128)
int8_mma_peak_pair_kernel(int n_tokens, int iters, int* status, int commits) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(8) uint64_t scratch_bar[2];
    __shared__ uint32_t s_tmem;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    for (int i = threadIdx.x; i < (n_tokens * 128) / 4; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
        reinterpret_cast<uint32_t*>(base)[i] = h;
    }
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&scratch_bar[0])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&scratch_bar[1])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    {
        const uint32_t lane_addr = (uint32_t)((threadIdx.x >> 5) * 32) << 16;
        for (int c = 0; c < 4; ++c) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                uint32_t h = (threadIdx.x * 64u + c * 16u + j) * 2654435761u + blockIdx.x * 7919u;
                h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
                r[j] = h;
            }
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                ::"r"(tmem + lane_addr + 256 + c * 16), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (threadIdx.x == 0 && rank == 0) {
        uint64_t bd = 0;
        bd |= (uint64_t)((smem_u32(base) & 0x3FFFFu) >> 4);
        bd |= (uint64_t)1 << 16;
        bd |= (uint64_t)(1024 >> 4) << 32;
        bd |= (uint64_t)1 << 46;
        bd |= (uint64_t)2 << 61;
        const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n_tokens >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
#pragma unroll 4
        for (int i = 0; i < iters; ++i) {
            const uint32_t a_addr = tmem + 256 + (uint32_t)(i & 7) * 8;
            const uint64_t b = bd + (uint64_t)((i & 3) * 2);
            asm volatile(
                "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
                ::"r"(tmem), "r"(a_addr), "l"(b), "r"(idesc), "r"(i > 0 ? 1u : 0u)
                : "memory");
            if ((i & 3) == 3)
                for (int c = 0; c < commits; ++c)
                    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                                 ::"r"(smem_u32(&scratch_bar[c & 1])), "h"((uint16_t)3) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     ::"r"(smem_u32(&bar)), "h"((uint16_t)3) : "memory");
    }
    if (threadIdx.x == 0) {     // both CTAs: bounded wait for the MMAs to retire
        const long long t0 = clock64();
        uint32_t done = 0;
        while (!done) {
            asm volatile("{\n\t.reg .pred P1;\n\tmbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\tselp.b32 %0, 1, 0, P1;\n\t}"
                         : "=r"(done) : "r"(smem_u32(&bar)), "r"(0u) : "memory");
            if (clock64() - t0 > 4000000000ll) { atomicExch(status, 1); break; }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}
#endif

}  // namespace

#ifdef MMF_EXPERIMENTS
int g_probe_commits = 0;   // mmf_tuning(MMF_TUNE_PROBE_COMMITS, n), experiments build only
int g_probe_issuers = 0;   // mmf_tuning(MMF_TUNE_PROBE_ISSUERS, 2): two issuing threads, experiments build only
#else
static constexpr int g_probe_commits = 0;
static constexpr int g_probe_issuers = 0;
#endif

extern "C" int mmf_int8_mma_peak(int n_tokens, int iters, int* status_dev, double* tops_host) {
    MMF_REQUIRE(status_dev && tops_host, MMF_ERR_BAD_ARG, "mmf_int8_mma_peak: null pointer");
    MMF_REQUIRE(n_tokens >= 16 && n_tokens <= 256 && n_tokens % 16 == 0 && iters > 0 && iters <= (1 << 25), MMF_ERR_BAD_SHAPE,
                "mmf_int8_mma_peak: n_tokens must be a multiple of 16 in [16,256], iters in (0, 32M]");
    int dev = 0, sms = 0;
    MMF_CUDA(cudaGetDevice(&dev));
    MMF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const size_t smem = 1024 + (size_t)n_tokens * 128;
    const int issuers = g_probe_issuers == 2 && n_tokens <= 128 ? 2 : 1;
    MMF_CUDA(cudaFuncSetAttribute(int8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(150 * 1024)));
    cudaEvent_t e0, e1;
    MMF_CUDA(cudaEventCreate(&e0));
    MMF_CUDA(cudaEventCreate(&e1));
    MMF_CUDA(cudaMemset(status_dev, 0, sizeof(int)));
    // 150 KB of shared memory per CTA keeps it at one CTA per SM (each allocates all of tensor memory)
#ifdef MMF_EXPERIMENTS
    if (g_probe_issuers == 3) {      // pair mode (cta_group::2): clusters of two CTAs, 256-row MMAs
        MMF_REQUIRE(n_tokens % 32 == 0, MMF_ERR_BAD_SHAPE, "mmf_int8_mma_peak(pair): n_tokens must be a multiple of 32");
        MMF_CUDA(cudaFuncSetAttribute(int8_mma_peak_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(150 * 1024)));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(sms & ~1));
        cfg.blockDim = dim3(128);
        cfg.dynamicSmemBytes = 150 * 1024;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        MMF_CUDA(cudaLaunchKernelEx(&cfg, int8_mma_peak_pair_kernel, n_tokens, 64, status_dev, g_probe_commits));
        MMF_CUDA(cudaEventRecord(e0));
        MMF_CUDA(cudaLaunchKernelEx(&cfg, int8_mma_peak_pair_kernel, n_tokens, iters, status_dev, g_probe_commits));
        MMF_CUDA(cudaEventRecord(e1));
        MMF_CUDA(cudaEventSynchronize(e1));
        MMF_LAUNCH_CHECK("int8_mma_peak_pair_kernel");
        float msp = 0.0f;
        MMF_CUDA(cudaEventElapsedTime(&msp, e0, e1));
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
        int stp = 0;
        MMF_CUDA(cudaMemcpy(&stp, status_dev, sizeof(int), cudaMemcpyDeviceToHost));
        MMF_REQUIRE(stp == 0, MMF_ERR_TIMEOUT, "mmf_int8_mma_peak(pair): the MMAs did not retire in time");
        *tops_host = 2.0 * 256.0 * n_tokens * 32.0 * (double)iters * (sms / 2) / ((double)msp * 1e-3) / 1e12;
        return MMF_OK;
    }
#endif
    int8_mma_peak_kernel<<<sms, 128, 150 * 1024>>>(n_tokens, 64, status_dev, g_probe_commits, issuers);     // warm-up
    MMF_CUDA(cudaEventRecord(e0));
    int8_mma_peak_kernel<<<sms, 128, 150 * 1024>>>(n_tokens, iters, status_dev, g_probe_commits, issuers);
    MMF_CUDA(cudaEventRecord(e1));
    MMF_CUDA(cudaEventSynchronize(e1));
    MMF_LAUNCH_CHECK("int8_mma_peak_kernel");
    float ms = 0.0f;
    MMF_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    int status = 0;
    MMF_CUDA(cudaMemcpy(&status, status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    MMF_REQUIRE(status == 0, MMF_ERR_TIMEOUT, "mmf_int8_mma_peak: the MMAs did not retire in time");
    (void)smem;
    *tops_host = 2.0 * 128.0 * n_tokens * 32.0 * (double)iters * sms / ((double)ms * 1e-3) / 1e12;
    return MMF_OK;
}


// =========================================================================================================
// Synchronisation costs that shape the decode step (measurement aid, no counterpart in the reference)
// =========================================================================================================
namespace {

constexpr long long SYNC_SPIN_LIMIT = 400000000ll;   // cycles: a wait that exceeds this gives up and sets the status word

__device__ __forceinline__ unsigned probe_ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void probe_red_release(unsigned* p) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}

// `iters` grid-wide barriers: every CTA adds 1 to a counter (release) and polls it (acquire) until all have arrived
__global__ void grid_barrier_probe_kernel(unsigned* counter, int iters, int* status) {
    const unsigned n = gridDim.x;
    bool ok = true;
    for (int k = 0; k < iters && ok; ++k) {
        __syncthreads();
        if (threadIdx.x == 0) {
            probe_red_release(counter);
            const long long t0 = clock64();
            while (probe_ld_acquire(counter) < (unsigned)(k + 1) * n) {
                if (clock64() - t0 > SYNC_SPIN_LIMIT) { *status = 1; ok = false; break; }
            }
        }
        ok = __syncthreads_and(ok);
    }
}

// two CTAs hand a flag back and forth `iters` times: release store -> acquire poll, one direction at a time
__global__ void signal_probe_kernel(unsigned* f0, unsigned* f1, int iters, int* status) {
    if (threadIdx.x != 0) return;
    for (int k = 1; k <= iters; ++k) {
        unsigned* mine = blockIdx.x == 0 ? f0 : f1;
        const unsigned* theirs = blockIdx.x == 0 ? f1 : f0;
        if (blockIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(mine), "r"((unsigned)k) : "memory");
        const long long t0 = clock64();
        while (probe_ld_acquire(theirs) < (unsigned)k)
            if (clock64() - t0 > SYNC_SPIN_LIMIT) { *status = 2; return; }
        if (blockIdx.x == 1) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(mine), "r"((unsigned)k) : "memory");
    }
}

// one link of a chain of dependent kernels: reads what its predecessor wrote, writes what its successor reads
__global__ void chain_link_kernel(const unsigned* in, unsigned* out) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) out[blockIdx.x & 31] = in[blockIdx.x & 31] + 1u;
}

// microseconds per kernel of a chain of `n` dependent launches of `blocks` x `threads` replayed from a CUDA graph, with or
// without the programmatic-dependent-launch attribute
int chain_us(int n, int blocks, int threads, bool pdl, unsigned* a, unsigned* b, double* us) {
    cudaStream_t st;
    MMF_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    MMF_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    for (int i = 0; i < n; ++i) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(threads);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl ? 1 : 0;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, chain_link_kernel, (const unsigned*)((i & 1) ? b : a), (i & 1) ? a : b);
        if (e != cudaSuccess) {
            cudaStreamEndCapture(st, &graph);
            if (graph) cudaGraphDestroy(graph);
            cudaStreamDestroy(st);
            return mmf_set_error(MMF_ERR_CUDA, "mmf_sync_probe: launch inside capture failed: %s", cudaGetErrorString(e));
        }
    }
    MMF_CUDA(cudaStreamEndCapture(st, &graph));
    MMF_CUDA(cudaGraphInstantiate(&exec, graph, 0));
    for (int i = 0; i < 3; ++i) MMF_CUDA(cudaGraphLaunch(exec, st));
    MMF_CUDA(cudaStreamSynchronize(st));
    cudaEvent_t e0, e1;
    MMF_CUDA(cudaEventCreate(&e0));
    MMF_CUDA(cudaEventCreate(&e1));
    MMF_CUDA(cudaEventRecord(e0, st));
    for (int i = 0; i < 10; ++i) MMF_CUDA(cudaGraphLaunch(exec, st));
    MMF_CUDA(cudaEventRecord(e1, st));
    MMF_CUDA(cudaStreamSynchronize(st));
    float ms = 0.0f;
    MMF_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    *us = ms * 1e3 / (10.0 * n);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaGraphExecDestroy(exec);
    cudaGraphDestroy(graph);
    cudaStreamDestroy(st);
    return MMF_OK;
}

}  // namespace

extern "C" int mmf_sync_probe(int iters, unsigned* scratch_dev, double* barrier_us_host, double* signal_us_host,
                              double* chain_pdl_us_host, double* chain_plain_us_host) {
    MMF_REQUIRE(scratch_dev && barrier_us_host && signal_us_host && chain_pdl_us_host && chain_plain_us_host, MMF_ERR_BAD_ARG,
                "mmf_sync_probe: null pointer");
    MMF_REQUIRE(iters > 0 && iters <= 100000, MMF_ERR_BAD_SHAPE, "mmf_sync_probe: iters must be in (0, 100000]");
    int dev = 0, sms = 0, coop = 0;
    MMF_CUDA(cudaGetDevice(&dev));
    MMF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MMF_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    MMF_REQUIRE(coop, MMF_ERR_ARCH, "mmf_sync_probe: the device does not support cooperative launches");
    cudaEvent_t e0, e1;
    MMF_CUDA(cudaEventCreate(&e0));
    MMF_CUDA(cudaEventCreate(&e1));
    // scratch: [0] barrier counter, [64] and [128] the two flags (separate cache lines), [192] status
    MMF_CUDA(cudaMemset(scratch_dev, 0, 256 * sizeof(unsigned)));
    unsigned* counter = scratch_dev;
    unsigned *f0 = scratch_dev + 64, *f1 = scratch_dev + 128;
    int* status = reinterpret_cast<int*>(scratch_dev + 192);
    float ms = 0.0f;
    {
        // co-resident by construction: a cooperative launch of one CTA per SM fails rather than run partially
        void* args[] = {&counter, &iters, &status};
        MMF_CUDA(cudaEventRecord(e0));
        MMF_CUDA(cudaLaunchCooperativeKernel((void*)grid_barrier_probe_kernel, dim3(sms), dim3(256), args, 0, 0));
        MMF_CUDA(cudaEventRecord(e1));
        MMF_CUDA(cudaEventSynchronize(e1));
        MMF_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        *barrier_us_host = ms * 1e3 / iters;
    }
    {
        void* args[] = {&f0, &f1, &iters, &status};
        MMF_CUDA(cudaEventRecord(e0));
        MMF_CUDA(cudaLaunchCooperativeKernel((void*)signal_probe_kernel, dim3(2), dim3(32), args, 0, 0));
        MMF_CUDA(cudaEventRecord(e1));
        MMF_CUDA(cudaEventSynchronize(e1));
        MMF_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        *signal_us_host = ms * 1e3 / iters / 2;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    int st = 0;
    MMF_CUDA(cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost));
    MMF_REQUIRE(st == 0, MMF_ERR_TIMEOUT, "mmf_sync_probe: a bounded wait gave up (status %d)", st);
    // a chain of 200 dependent one-CTA-per-SM kernels: what a launch boundary costs with and without the
    // programmatic-dependent-launch attribute
    int rc = chain_us(200, sms, 256, true, scratch_dev + 64, scratch_dev + 128, chain_pdl_us_host);
    if (rc != MMF_OK) return rc;
    rc = chain_us(200, sms, 256, false, scratch_dev + 64, scratch_dev + 128, chain_plain_us_host);
    return rc;
}
