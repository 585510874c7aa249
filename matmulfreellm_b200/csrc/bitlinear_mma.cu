// BitLinear on the 5th-generation tensor cores (tcgen05, kind::i8, int32 accumulators in TMEM).
//
// Orientation ("swap-AB"): the MMA's M dimension is a 128-row WEIGHT tile, its N dimension is
// the token rows (16..256 per instruction), so one weight tile meets every token with a single
// pass over its 2-bit stream.  The weight operand never exists as int8 in memory: packed 16-byte
// pieces (64 weights) arrive in shared memory by bulk TMA, each of 128 threads expands the piece
// of "its" weight row in registers into 16 x 32-bit words of int8 and writes them with
// tcgen05.st straight into tensor memory, where the MMA reads its A operand (A-from-TMEM form).
// The token operand (int8 activation codes, K-major) is fetched by tiled TMA with the 128-byte
// swizzle into a shared-memory ring and read through a UMMA shared-memory descriptor.
//
// Warp roles (352 threads): warps 0-7 unpack — two groups of four warps that alternate 128-K
// stages, lane <-> TMEM lane <-> weight row — and later run the epilogue; warp 8 = activation-tile
// TMA producer; warp 9 = TMEM owner + MMA issuer; warp 10 = packed-weight TMA producer.  Three
// rings (packed weights in smem, unpacked A stages in TMEM, activation tiles in smem) are
// synchronised with mbarriers; every wait is bounded and reports through a status word instead
// of hanging.  The weight stream does not depend on the preceding kernel, so it is started
// before the grid-dependency wait (programmatic dependent launch).
//
// Weights are stored biased (+1); sum_k (t+1)*x = acc + rowsum(x) and the epilogue subtracts the
// per-token code sum.  For few tokens the K range is split over the CTAs of a thread-block cluster
// (2, 4 or 8) to fill the GPU; each CTA parks its partial int32 tile in its own shared memory and,
// after a cluster barrier, reduces its share of the token columns over its peers' tiles through
// distributed shared memory (integer adds: deterministic) and dequantises them.
#include <cuda.h>

#include "bitlinear.cuh"

namespace {

constexpr int NUM_UNPACK_WARPS = 8;
constexpr int UNPACK_THREADS = NUM_UNPACK_WARPS * 32;
constexpr int WARP_B = 8, WARP_MMA = 9, WARP_W = 10;
constexpr int MM_THREADS = 11 * 32;
// ring depths are chosen per launch (MmaParams); these are the capacities of the barrier table
constexpr int MAX_SA = 16;        // A stages (128 K = 32 TMEM columns each) in flight
constexpr int MAX_SB = 32;        // activation stages (128 K each)
constexpr int MAX_SW = 32;        // packed-weight stages (128 K = 4 KB each)
constexpr int W_STAGE_BYTES = 2 * MMF_TILE_ROWS * 16;  // two 64-K chunks
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;

struct MmaParams {
    int KC;              // K / 64
    int n_tiles, group_tiles;
    int NT;              // token rows per tile (multiple of 16, <= 256)
    int ksplit;          // CTAs sharing one output tile along K
    int stages_per_cta;  // 128-K stages per CTA
    int tmem_cols;       // power of two >= nacc*NT + SA*32
    int wt;              // weight tiles (128 rows each) one CTA multiplies against each activation stage: 1 or 2
    int nacc;            // independent accumulators (NT columns each) that consecutive MMAs rotate through
    int SA, SB, SW;      // ring depths: unpacked-A stages in TMEM, activation stages, packed-weight stages
    uint32_t idesc;
};

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

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred P;\n\t.reg .b32 r;\n\t"
        "elect.sync r|P, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, P;\n\t}"
        : "=r"(pred));
    return pred != 0;
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

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// optional phase trace of CTA (0,0,0): armed by writing MMF_TRACE_MAGIC into workspace word 1
constexpr int MMF_TRACE_MAGIC = 0x7ace;
__device__ __forceinline__ void trace_mark(long long* trace, int slot) {
    if (trace) trace[slot] = clock64();
}

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

// barrier table: index ranges inside one uint64 array
constexpr int BAR_B_FULL = 0, BAR_B_EMPTY = BAR_B_FULL + MAX_SB, BAR_W_FULL = BAR_B_EMPTY + MAX_SB,
              BAR_W_EMPTY = BAR_W_FULL + MAX_SW, BAR_A_FULL = BAR_W_EMPTY + MAX_SW, BAR_A_EMPTY = BAR_A_FULL + MAX_SA,
              BAR_ACC = BAR_A_EMPTY + MAX_SA, NUM_BARS = BAR_ACC + 1;

__device__ __forceinline__ uint32_t bar_count(int i) {
    // arrivals per phase: the 128 threads of one unpack group for "weights consumed" and "A stage written",
    // one (producer's expect_tx arrive or a tcgen05.commit) for everything else
    return (i >= BAR_W_EMPTY && i < BAR_A_EMPTY) ? 128u : 1u;
}


__device__ __forceinline__ void st_peer_v4(void* my_smem_addr, uint32_t peer_rank, const int4& v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem_addr)), "r"(peer_rank));
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Finish 8 consecutive outputs (rows n..n+7 of the weight tile) of token m: subtract the +1 bias, dequantise,
// convert and store as one 16-byte (2-byte dtypes) or two 16-byte (fp32) stores when the row allows it.
__device__ __forceinline__ void finish8(const BitLinearArgs& a, int32_t (&acc)[8], int m, int n, int rowsum, float scale) {
    if (n >= a.N) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] -= rowsum;
    const bool full = n + 8 <= a.N;
    if (a.acc_out) {
        int32_t* dst = a.acc_out + (int64_t)m * a.N + n;
        if (full && (a.N & 3) == 0) {
            reinterpret_cast<int4*>(dst)[0] = make_int4(acc[0], acc[1], acc[2], acc[3]);
            reinterpret_cast<int4*>(dst)[1] = make_int4(acc[4], acc[5], acc[6], acc[7]);
        } else {
            for (int i = 0; i < 8 && n + i < a.N; ++i) dst[i] = acc[i];
        }
    }
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __fmul_rn((float)acc[i], scale);
    const int64_t off = (int64_t)m * a.ld_out + n;
    if (a.out_dtype == MMF_F32) {
        float* dst = reinterpret_cast<float*>(a.out) + off;
        if (full && (a.ld_out & 3) == 0) {
            reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
        } else {
            for (int i = 0; i < 8 && n + i < a.N; ++i) dst[i] = f[i];
        }
    } else {
        uint32_t w[4];
        if (a.out_dtype == MMF_BF16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        uint16_t* dst = reinterpret_cast<uint16_t*>(a.out) + off;
        if (full && (a.ld_out & 7) == 0) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            const uint16_t* h = reinterpret_cast<const uint16_t*>(w);
            for (int i = 0; i < 8 && n + i < a.N; ++i) dst[i] = h[i];
        }
    }
}

__global__ void __launch_bounds__(MM_THREADS, 2)
bitlinear_mma_kernel(const __grid_constant__ CUtensorMap q_map, BitLinearArgs a, MmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    // carve (1024-byte aligned for the 128-byte swizzle atoms): [activation ring | packed-weight ring | landing zone]
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_stage_bytes = p.NT * 128;
    uint8_t* b_ring = base;
    const int SA = p.SA, SB = p.SB, SW = p.SW;
    uint8_t* w_ring = base + SB * b_stage_bytes;
    int32_t* stg = reinterpret_cast<int32_t*>(b_ring);   // [NT][128] this CTA's int32 tile; reuses the idle activation ring
    // split-K landing zone [ksplit][NT/ksplit][128] int32: peers push the token columns this CTA finishes
    int32_t* part = reinterpret_cast<int32_t*>(w_ring + SW * W_STAGE_BYTES);

    __shared__ __align__(8) uint64_t bars[NUM_BARS];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ float s_dq[256];
    __shared__ int s_rs[256];

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int ks = blockIdx.x, tile = blockIdx.y * p.wt, mt = blockIdx.z;
    const int ntile = min(p.wt, p.n_tiles - tile);   // weight tiles this CTA owns (2 = dual-tile mode for large M)
    long long* trace = nullptr;
    if (tid == 0 && a.ws && a.ws[1] == MMF_TRACE_MAGIC && (blockIdx.x | blockIdx.y | blockIdx.z) == 0)
        trace = reinterpret_cast<long long*>(a.ws + 8);
    trace_mark(trace, 0);
    pdl_trigger();   // the next kernel may start its own prologue (and weight stream) right away
    const int g = tile / p.group_tiles;
    const int m0 = mt * p.NT;
    const int stage0 = ks * p.stages_per_cta;
    const int total_stages = (p.KC + 1) / 2;
    const int nstages = min(p.stages_per_cta, total_stages - stage0);   // >= 1 by construction

    static_assert(NUM_BARS <= MM_THREADS, "one thread initialises one barrier");
    if (tid < NUM_BARS) mbar_init(&bars[tid], bar_count(tid));
    if (tid == NUM_BARS) s_abort = 0;
    if (warp == WARP_MMA) tmem_alloc(&s_tmem_base, (uint32_t)p.tmem_cols);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // cluster barrier #1 (arrive now, wait before the first remote store): a peer's shared memory may only be
    // written once that peer is known to be running
    if (p.ksplit > 1) cluster_arrive();
    trace_mark(trace, 1);
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t tmem_a = tmem_base + (uint32_t)(p.wt * p.nacc * p.NT);   // A stages (32 columns each) follow the accumulators
    volatile int* abort_flag = &s_abort;

    // ring cursors advance by increment-and-wrap (no division in the hot loops); `ph` is the barrier phase bit
    struct Ring {
        int slot, ph, depth;
        __device__ __forceinline__ void next() { if (++slot == depth) { slot = 0; ph ^= 1; } }
        __device__ __forceinline__ void next2() { next(); next(); }
    };

    if (warp == WARP_W) {
        // ------------------------------------------------------------ packed weights (bulk TMA)
        // Weights do not depend on the preceding kernel: their stream starts before the grid dependency wait.
        if (elect_one()) {
            Ring w{0, 0, SW};
            for (int i = 0; i < nstages; ++i, w.next()) {
                const uint32_t bytes = (uint32_t)min(2, p.KC - (stage0 + i) * 2) * (MMF_TILE_ROWS * 16);
                for (int t = 0; t < ntile; ++t) {
                    const int slot = t * SW + w.slot;
                    if (!mbar_wait(&bars[BAR_W_EMPTY + slot], w.ph ^ 1, abort_flag)) { i = nstages; break; }
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.packed) +
                                         ((int64_t)(tile + t) * p.KC + (int64_t)(stage0 + i) * 2) * (MMF_TILE_ROWS * 16);
                    mbar_expect_tx(&bars[BAR_W_FULL + slot], bytes);
                    bulk_load_1d(w_ring + slot * W_STAGE_BYTES, src, bytes, &bars[BAR_W_FULL + slot]);
                }
            }
        }
    } else if (warp == WARP_B) {
        // ------------------------------------------------------------ activation tiles (TMA, swizzled)
        pdl_wait();   // the codes are the preceding kernel's output
        if (elect_one()) {
            Ring bq{0, 0, SB};
            const int y = g * a.M + m0;
            for (int i = 0; i < nstages; ++i, bq.next()) {
                if (!mbar_wait(&bars[BAR_B_EMPTY + bq.slot], bq.ph ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars[BAR_B_FULL + bq.slot], (uint32_t)b_stage_bytes);
                tma_load_2d(b_ring + bq.slot * b_stage_bytes, &q_map, &bars[BAR_B_FULL + bq.slot], (stage0 + i) * 128, y);
            }
        }
    } else if (warp == WARP_MMA) {
        // ------------------------------------------------------------ MMA issue
        // One thread feeds the tensor core; the loop carries no division and builds descriptors by addition so
        // that it stays well under the ~88 (N <= 128) / 130 (N = 256) cycles one MMA occupies the pipe.
        if (elect_one()) {
            Ring bq{0, 0, SB}, aq{0, 0, SA};
            const uint64_t b_desc0 = make_b_desc(smem_u32(b_ring));
            const uint32_t b_desc_step = (uint32_t)b_stage_bytes >> 4;
            // consecutive MMAs rotate through `nacc` independent accumulators; the epilogue adds them (exact)
            int acc = 0;
            uint32_t started = 0;     // MMAs issued so far, saturating at nacc: the first use of an accumulator overwrites
            const uint32_t nacc = (uint32_t)p.nacc, NTc = (uint32_t)p.NT;
            bool live = true;
            for (int i = 0; i < nstages && live; ++i, bq.next(), aq.next()) {
                if (!mbar_wait(&bars[BAR_B_FULL + bq.slot], bq.ph, abort_flag)) break;
                const uint64_t bd = b_desc0 + (uint64_t)(bq.slot * b_desc_step);
                const int nmma = min(2, p.KC - (stage0 + i) * 2) * 2;
                for (int t = 0; t < ntile; ++t) {
                    const int slot = t * SA + aq.slot;
                    if (!mbar_wait(&bars[BAR_A_FULL + slot], aq.ph, abort_flag)) { live = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = tmem_a + slot * 32;
                    if (p.wt == 2) {
                        // dual-tile: one activation stage feeds two 128-row weight tiles (accumulators t*NT)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (k < nmma) mma_i8_ts(tmem_base + t * NTc, a_addr + k * 8, bd + (uint64_t)(k * 2), p.idesc, (i | k) != 0 ? 1u : 0u);
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            if (k < nmma) {
                                mma_i8_ts(tmem_base + acc * NTc, a_addr + k * 8, bd + (uint64_t)(k * 2), p.idesc, started >= nacc ? 1u : 0u);
                                if (++acc == (int)nacc) acc = 0;
                                if (started < nacc) ++started;
                            }
                        }
                    }
                    tc_commit(&bars[BAR_A_EMPTY + slot]);   // frees the A stage when these MMAs retire
                }
                tc_commit(&bars[BAR_B_EMPTY + bq.slot]);
            }
            tc_commit(&bars[BAR_ACC]);
        }
    } else {
        // ------------------------------------------------------------ unpack (two groups of 4 warps), then epilogue
        const int qd = warp & 3, gp = warp >> 2;
        const int row = qd * 32 + lane;                      // weight row in the tile == TMEM lane
        const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
        bool ok = true;
        // one weight tile per CTA: the two groups alternate stages; two tiles: group gp owns tile gp, every stage
        Ring w{0, 0, SW}, aq{0, 0, SA};
        const bool dual = p.wt == 2;
        if (!dual && gp) { w.next(); aq.next(); }
        const int w_off = dual ? gp * SW : 0, a_off = dual ? gp * SA : 0;
        const int i_step = dual ? 1 : 2;
        for (int i = dual ? 0 : gp; i < nstages && ok && (!dual || gp < ntile); i += i_step) {
            const int ws = w_off + w.slot, as = a_off + aq.slot;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars[BAR_W_FULL + ws], w.ph, abort_flag));   // warp-uniform
            if (!ok) break;
            if (i == 0) trace_mark(trace, 2);
            const int nch = min(2, p.KC - (stage0 + i) * 2);
            const uint8_t* wsrc = w_ring + ws * W_STAGE_BYTES + row * 16;
            uint4 wv[2];
            wv[0] = *reinterpret_cast<const uint4*>(wsrc);
            wv[1] = nch > 1 ? *reinterpret_cast<const uint4*>(wsrc + MMF_TILE_ROWS * 16) : wv[0];
            mbar_arrive(&bars[BAR_W_EMPTY + ws]);             // the packed bytes are in registers now
            ok = __all_sync(0xffffffffu, mbar_wait(&bars[BAR_A_EMPTY + as], aq.ph ^ 1, abort_flag));
            if (!ok) break;   // uniform per warp: the .sync.aligned tcgen05 ops below need the whole warp
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (h < nch) {
                    const uint32_t words[4] = {wv[h].x, wv[h].y, wv[h].z, wv[h].w};
                    uint32_t r[16];
#pragma unroll
                    for (int w4 = 0; w4 < 4; ++w4)
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4) r[w4 * 4 + k4] = (words[w4] >> (2 * k4)) & 0x03030303u;
                    tmem_st16(tmem_a + lane_addr + as * 32 + h * 16, r);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[BAR_A_FULL + as]);
            if (dual) { w.next(); aq.next(); } else { w.next2(); aq.next2(); }
        }
        trace_mark(trace, 3);

        // ---- epilogue phase A: accumulator tile TMEM -> shared memory [token][row]
        pdl_wait();                                       // dq / rowsum come from the preceding kernel
        for (int i = tid; i < p.NT; i += UNPACK_THREADS) {
            const int m = m0 + i;
            const bool in = m < a.M;
            s_dq[i] = in ? a.dq[(int64_t)g * a.M + m] : 0.0f;
            s_rs[i] = in ? a.rowsum[(int64_t)g * a.M + m] : 0;
        }
        ok = __all_sync(0xffffffffu, ok && mbar_wait(&bars[BAR_ACC], 0, abort_flag));
        tc_fence_after();
        trace_mark(trace, 4);
        if (ok) {
            const int ngroups = p.NT >> 4;
            if (dual) {
                // group gp stages the accumulator of tile gp: stg[(gp*NT + column)][row]
                if (gp < ntile) {
                    for (int gi = 0; gi < ngroups; ++gi) {
                        uint32_t v0[16];
                        tmem_ld16(tmem_base + lane_addr + gp * p.NT + gi * 16, v0);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) stg[(gp * p.NT + gi * 16 + j) * MMF_TILE_ROWS + row] = (int32_t)v0[j];
                    }
                }
            } else {
                const int total_mma = (min(p.KC, (stage0 + nstages) * 2) - stage0 * 2) * 2;   // MMAs this CTA issued
                const int nused = min(p.nacc, total_mma);                                      // accumulators that hold data
                for (int gi = gp; gi < ngroups; gi += 2) {        // groups of 16 columns, alternating between the warp groups
                    uint32_t v0[16], v1[16];
                    tmem_ld16(tmem_base + lane_addr + gi * 16, v0);
                    for (int acc = 1; acc < nused; ++acc) {       // fold the other accumulators in
                        tmem_ld16(tmem_base + lane_addr + acc * p.NT + gi * 16, v1);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) v0[j] += v1[j];
                    }
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) stg[(gi * 16 + j) * MMF_TILE_ROWS + row] = (int32_t)v0[j];
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(UNPACK_THREADS) : "memory");   // the 8 epilogue warps only
        trace_mark(trace, 5);

        // ---- phase B: 16 threads per token column, 8 consecutive weight rows each
        const int cth = tid >> 4, n8 = (tid & 15) * 8;
        const int n = tile * MMF_TILE_ROWS + n8;
        const float wsc = a.w_scale[g];
        if (p.ksplit == 1) {
            if (ok) {
                for (int t = 0; t < ntile; ++t) {
                    const int32_t* src = stg + t * p.NT * MMF_TILE_ROWS;
                    for (int c = cth; c < p.NT; c += UNPACK_THREADS / 16) {
                        const int m = m0 + c;
                        if (m >= a.M) break;
                        const int4 x0 = *reinterpret_cast<const int4*>(src + c * MMF_TILE_ROWS + n8);
                        const int4 x1 = *reinterpret_cast<const int4*>(src + c * MMF_TILE_ROWS + n8 + 4);
                        int32_t acc[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
                        finish8(a, acc, m, n + t * MMF_TILE_ROWS, s_rs[c], __fmul_rn(s_dq[c], wsc));
                    }
                }
            }
        } else {
            const int per = p.NT / p.ksplit;                  // token columns each CTA of the cluster finishes
            cluster_wait();                                   // barrier #1: every CTA of the cluster is running
            if (ok) {
                // push the columns owned by peer o into its landing zone, slot [my rank]
                const int vecs = per * (MMF_TILE_ROWS / 4);   // int4 pieces per slice
                for (int o = 0; o < p.ksplit; ++o) {
                    if (o == ks) continue;
                    const int4* src = reinterpret_cast<const int4*>(stg + o * per * MMF_TILE_ROWS);
                    int4* dst = reinterpret_cast<int4*>(part + ks * per * MMF_TILE_ROWS);
                    for (int idx = tid; idx < vecs; idx += UNPACK_THREADS) st_peer_v4(dst + idx, (uint32_t)o, src[idx]);
                }
            }
            cluster_arrive();                                 // barrier #2 orders all pushes before the owners' reads
            cluster_wait();
            trace_mark(trace, 6);
            if (ok && !*abort_flag) {
                for (int cl = cth; cl < per; cl += UNPACK_THREADS / 16) {
                    const int c = ks * per + cl;
                    const int m = m0 + c;
                    if (m >= a.M) break;
                    const int4 x0 = *reinterpret_cast<const int4*>(stg + c * MMF_TILE_ROWS + n8);
                    const int4 x1 = *reinterpret_cast<const int4*>(stg + c * MMF_TILE_ROWS + n8 + 4);
                    int32_t acc[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int peer = 0; peer < 8; ++peer) {
                        if (peer < p.ksplit && peer != ks) {
                            const int4 y0 = *reinterpret_cast<const int4*>(part + (peer * per + cl) * MMF_TILE_ROWS + n8);
                            const int4 y1 = *reinterpret_cast<const int4*>(part + (peer * per + cl) * MMF_TILE_ROWS + n8 + 4);
                            acc[0] += y0.x; acc[1] += y0.y; acc[2] += y0.z; acc[3] += y0.w;
                            acc[4] += y1.x; acc[5] += y1.y; acc[6] += y1.z; acc[7] += y1.w;
                        }
                    }
                    finish8(a, acc, m, n, s_rs[c], __fmul_rn(s_dq[c], wsc));
                }
            }
        }
        trace_mark(trace, 7);
    }

    if (p.ksplit > 1 && warp >= NUM_UNPACK_WARPS) {   // the three service warps take part in both cluster barriers
        cluster_wait();
        cluster_arrive();
        cluster_wait();
    }

    // teardown: everyone meets, TMEM goes back; on the error path give copies in flight time to land first
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
    tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

}  // namespace

// tuning overrides (0 = automatic), see mmf_tuning()
static int g_force_ksplit = 0, g_force_nt = 0, g_force_deep = 0, g_force_wt = 0, g_force_sb = 0, g_force_sa = 0, g_force_sw = 0;

extern "C" int mmf_tuning(int knob, int value) {
    switch (knob) {
        case MMF_TUNE_KSPLIT: g_force_ksplit = value; return MMF_OK;
        case MMF_TUNE_TOKEN_TILE: g_force_nt = value; return MMF_OK;
        case MMF_TUNE_DEEP_RING: g_force_deep = value; return MMF_OK;
        case MMF_TUNE_WEIGHT_TILES: g_force_wt = value; return MMF_OK;
        case MMF_TUNE_B_STAGES: g_force_sb = value; return MMF_OK;
        case MMF_TUNE_A_STAGES: g_force_sa = value; return MMF_OK;
        case MMF_TUNE_W_STAGES: g_force_sw = value; return MMF_OK;
        default: return mmf_set_error(MMF_ERR_BAD_ARG, "mmf_tuning: unknown knob %d", knob);
    }
}

namespace {

// Pick token tile, K split and ring depths.  Two regimes:
//  * "deep ring" (few tokens, no K split): the CTA owns all of TMEM (512 columns), so up to 14 unpacked A
//    stages plus a 24-stage packed ring hold most of a weight tile BEFORE the activations exist — under
//    programmatic dependent launch the weight stream and its unpacking overlap the preceding kernels, and
//    what is left after the dependency wait is the activation load, the MMAs and the epilogue;
//  * "split" (more tokens / few weight tiles): 4 A stages, K split over a cluster when that fills the GPU.
// The estimate below is a latency model in microseconds fitted to measured phase times of this kernel.
bool choose_config(const BitLinearArgs& a, MmaParams& best, size_t& best_smem) {
    const int KC = a.K / MMF_TILE_K;
    const int n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const int total_stages = (KC + 1) / 2;
    double best_cost = 1e30;
    bool found = false;
    int nts[3], n_nt = 0;
    if (a.M <= 128) nts[n_nt++] = ((a.M + 15) / 16) * 16;
    else { nts[n_nt++] = 128; nts[n_nt++] = 256; }
    for (int ni = 0; ni < n_nt; ++ni) {
        const int NT = nts[ni];
        if (g_force_nt && NT != g_force_nt) continue;
        const int m_tiles = (a.M + NT - 1) / NT;
        for (int ks = 1; ks <= 8; ks *= 2) {
            if (ks > 1 && (NT > 128 || ks > total_stages)) break;
            if (g_force_ksplit && ks != g_force_ksplit) continue;
            const int stages = (total_stages + ks - 1) / ks;
            if (ks > 1 && stages * (ks - 1) >= total_stages) continue;   // every CTA must own >= 1 stage
            for (int mode = 0; mode <= 2; ++mode) {          // 0 = plain, 1 = deep ring, 2 = two weight tiles per CTA
                const int deep = mode == 1;
                if (deep && (ks != 1 || NT > 64 || g_force_deep != 1)) continue;   // deep ring only on request
                const int group_tiles = n_tiles / a.groups;
                if (mode == 2 && (ks != 1 || NT != 128 || n_tiles < 2 || (a.groups > 1 && group_tiles % 2) || g_force_wt == 1)) continue;
                if (mode != 2 && g_force_wt == 2 && ks == 1 && NT == 128 && n_tiles >= 2) continue;
                if (g_force_deep == 1 && !deep && ks == 1 && NT <= 64) continue;
                if (g_force_deep == 2 && deep) continue;
                MmaParams p;
                p.KC = KC; p.n_tiles = n_tiles; p.group_tiles = group_tiles; p.NT = NT; p.ksplit = ks; p.wt = mode == 2 ? 2 : 1;
                p.stages_per_cta = stages;
                size_t smem;
                int occ;
                if (deep) {
                    p.tmem_cols = 512;
                    p.nacc = 256 / NT < 8 ? 256 / NT : 8;
                    p.SA = (512 - p.nacc * NT) / 32; if (p.SA > MAX_SA) p.SA = MAX_SA;
                    p.SW = stages < 24 ? stages : 24;
                    const size_t room = 220 * 1024 - (size_t)p.SW * W_STAGE_BYTES;
                    p.SB = (int)(room / ((size_t)NT * 128));
                    if (p.SB > stages) p.SB = stages;
                    if (p.SB > MAX_SB) p.SB = MAX_SB;
                    smem = 1024 + (size_t)p.SB * NT * 128 + (size_t)p.SW * W_STAGE_BYTES;
                    if (smem < 120 * 1024) smem = 120 * 1024;   // one CTA per SM: it holds all 512 TMEM columns
                    occ = 1;
                } else if (mode == 2) {
                    p.SA = 4; p.SB = 4; p.SW = 8; p.nacc = 1;
                    p.tmem_cols = 512;                              // 2 x 128 accumulator columns + 2 x 4 x 32 A columns
                    smem = 1024 + (size_t)p.SB * NT * 128 + (size_t)2 * p.SW * W_STAGE_BYTES;
                    occ = 1;
                } else {
                    p.SA = 4; p.SB = 4; p.SW = NT >= 128 ? 8 : 12;   // 8 keeps a 128-token tile under half an SM's shared memory
                    p.nacc = NT >= 128 ? 1 : (128 / NT < 4 ? 128 / NT : 4);
                    if (g_force_sb) p.SB = g_force_sb < MAX_SB ? g_force_sb : MAX_SB;
                    if (g_force_sa) p.SA = (g_force_sa < MAX_SA ? g_force_sa : MAX_SA) & ~1;   // the two unpack groups alternate slots
                    if (g_force_sw) p.SW = (g_force_sw < MAX_SW ? g_force_sw : MAX_SW) & ~1;
                    if (p.SA < 2 || p.SW < 2 || p.SB < 1 || p.nacc * NT + p.SA * 32 > 512) continue;
                    // the epilogue parks the int32 tile [NT][128] in the (then idle) rings
                    if ((size_t)p.SB * NT * 128 + (ks == 1 ? (size_t)p.SW * W_STAGE_BYTES : 0) < (size_t)NT * 512) continue;
                    int cols = 32;
                    while (cols < p.nacc * NT + p.SA * 32) cols *= 2;
                    p.tmem_cols = cols;
                    smem = 1024 + (size_t)p.SB * NT * 128 + (size_t)p.SW * W_STAGE_BYTES + (ks > 1 ? (size_t)NT * MMF_TILE_ROWS * 4 : 0);
                    occ = (smem <= 110 * 1024 && cols <= 256) ? 2 : 1;
                }
                if (smem > 227 * 1024) continue;
                const int64_t ctas = (int64_t)((n_tiles + p.wt - 1) / p.wt) * m_tiles * ks;
                const int64_t waves = (ctas + 148 * occ - 1) / (148 * occ);
                // fitted to measured phase times (us): per 128-K stage 4 MMAs of >= 88 cycles each (130 at 256 token
                // columns) plus issue overhead; fixed launch/set-up/first-TMA latency; epilogue; cluster reduction
                const double t_stage = mode == 2 ? 0.90 : NT > 128 ? 0.30 : 0.24;   // (two tiles per CTA measured slower: kept for experiments)
                double t = 2.5 + stages * t_stage + 0.5 + p.wt * NT * 0.012;
                if (ks > 1) t += 1.5 + NT * 0.012;
                const double cost = waves * t;
                if (cost < best_cost) { best_cost = cost; best = p; best_smem = smem; found = true; }
            }
        }
    }
    return found;
}

}  // namespace

int bitlinear_mma_launch(const BitLinearArgs& a, cudaStream_t st) {
    MmaParams p;
    size_t smem = 0;
    MMF_REQUIRE(choose_config(a, p, smem), MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): no kernel configuration fits M=%d N=%d K=%d", a.M,
                a.N, a.K);
    const int m_tiles = (a.M + p.NT - 1) / p.NT;
    // instruction descriptor: D=S32, A=S8 (TMEM), B=S8 (smem, K-major), M=128, N=NT
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    EncodeTiledFn encode = get_encode_tiled();
    MMF_REQUIRE(encode != nullptr, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap q_map;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.groups * (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.K};
    const cuuint32_t box[2] = {128u, (cuuint32_t)p.NT};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult cr = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(a.q), gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MMF_REQUIRE(cr == CUDA_SUCCESS, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled failed (%d)", (int)cr);

    MMF_CUDA(cudaFuncSetAttribute(bitlinear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((unsigned)p.ksplit, (unsigned)((p.n_tiles + p.wt - 1) / p.wt), (unsigned)m_tiles);
    MMF_REQUIRE(m_tiles <= 65535 && p.n_tiles <= 65535, MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): problem too large");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    MMF_CUDA(cudaLaunchKernelEx(&cfg, bitlinear_mma_kernel, q_map, a, p));
    MMF_LAUNCH_CHECK("bitlinear_mma_kernel");
    return MMF_OK;
}
