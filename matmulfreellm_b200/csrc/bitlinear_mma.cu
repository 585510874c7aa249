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
// (2, 4 or 8) to fill the GPU; each CTA owns a share of the token columns, writes the partial int32
// sums of every other share from its registers straight into the owner's shared memory (distributed
// shared memory stores) and, after one cluster barrier, adds up the slots it received (integer adds:
// deterministic) and dequantises them.
#include <cuda.h>

#include "bitlinear.cuh"
#include "tensor_map.cuh"
#include "tcgen05.cuh"

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

#ifndef MMF_ASYNC_REDUCE_DEFAULT
#define MMF_ASYNC_REDUCE_DEFAULT 1
#endif

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
    int merged;          // SA == SB and both rings share one full / one empty barrier per stage (one wait, one commit)
    int async_red;       // split-K: partial sums travel as st.async with the byte count credited to the owner's mbarrier,
                         // each owner waits for its own bytes only (no second cluster barrier)
    uint32_t idesc;
};

// ---------------------------------------------------
constexpr int BAR_B_FULL = 0, BAR_B_EMPTY = BAR_B_FULL + MAX_SB, BAR_W_FULL = BAR_B_EMPTY + MAX_SB,
              BAR_W_EMPTY = BAR_W_FULL + MAX_SW, BAR_A_FULL = BAR_W_EMPTY + MAX_SW, BAR_A_EMPTY = BAR_A_FULL + MAX_SA,
              BAR_ACC = BAR_A_EMPTY + MAX_SA, BAR_RED = BAR_ACC + 1, NUM_BARS = BAR_RED + 1;

__device__ __forceinline__ uint32_t bar_count(int i, int merged) {
    // merged rings: a stage's "full" barrier also takes the activation producer's expect_tx arrival
    if (merged && i >= BAR_A_FULL && i < BAR_A_EMPTY) return 129u;
    // arrivals per phase: the 128 threads of one unpack group for "weights consumed" and "A stage written",
    // one (producer's expect_tx arrive or a tcgen05.commit) for everything else
    return (i >= BAR_W_EMPTY && i < BAR_A_EMPTY) ? 128u : 1u;
}


// address of this CTA's shared-memory location `my_smem_addr` in CTA `peer_rank` of the cluster
__device__ __forceinline__ uint32_t peer_addr(const void* my_smem_addr, uint32_t peer_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem_addr)), "r"(peer_rank));
    return remote;
}
__device__ __forceinline__ void st_cluster_b32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// 4 bytes into a peer's shared memory; on arrival the peer's mbarrier is credited with the 4 bytes
__device__ __forceinline__ void st_async_b32(uint32_t cluster_addr, uint32_t v, uint32_t cluster_mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(cluster_addr), "r"(v),
                 "r"(cluster_mbar)
                 : "memory");
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
#ifdef MMF_EXPERIMENTS
    __shared__ long long* s_trace;
    if (tid == 0) s_trace = (a.ws && a.ws[1] == MMF_TRACE_MAGIC && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) ? trace_record(a.ws) : nullptr;
    long long* const trace = tid == 0 ? s_trace : nullptr;
#else
    long long* const trace = nullptr;
#endif
    trace_mark(trace, 0);
    pdl_trigger();   // the next kernel may start its own prologue (and weight stream) right away
    if (tid == WARP_B * 32) tma_prefetch_map(&q_map);   // descriptor ready before the dependency wait ends
    const int g = tile / p.group_tiles;
    const int m0 = mt * p.NT;
    const int stage0 = ks * p.stages_per_cta;
    const int total_stages = (p.KC + 1) / 2;
    const int nstages = min(p.stages_per_cta, total_stages - stage0);   // >= 1 by construction

    static_assert(NUM_BARS <= MM_THREADS, "one thread initialises one barrier");
    if (tid < NUM_BARS) mbar_init(&bars[tid], bar_count(tid, p.merged));
    if (tid == NUM_BARS) s_abort = 0;
    if (warp == WARP_MMA) tmem_alloc(&s_tmem_base, (uint32_t)p.tmem_cols);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // split-K with asynchronous pushes: this CTA will receive NT/ksplit token columns x 128 rows x 4 bytes from each of the
    // ksplit CTAs of its cluster (its own share included); credits that arrive before this line only make the count
    // negative for a moment
    if (p.ksplit > 1 && p.async_red && tid == 0) mbar_expect_tx(&bars[BAR_RED], (uint32_t)(p.NT * MMF_TILE_ROWS * 4));
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
                uint64_t* empty = &bars[(p.merged ? BAR_A_EMPTY : BAR_B_EMPTY) + bq.slot];
                uint64_t* full = &bars[(p.merged ? BAR_A_FULL : BAR_B_FULL) + bq.slot];
                if (!mbar_wait(empty, bq.ph ^ 1, abort_flag)) break;
                mbar_expect_tx(full, (uint32_t)b_stage_bytes);
                tma_load_2d(b_ring + bq.slot * b_stage_bytes, &q_map, full, (stage0 + i) * 128, y);
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
            int i = 0;
#ifdef MMF_EXPERIMENTS
            long long* const mtrace = s_trace;     // written before the __syncthreads above
#else
            long long* const mtrace = nullptr;
#endif
            if (p.wt == 1 && (nacc == 1 || nacc == 2 || nacc == 4)) {
                // lean path (one weight tile, whole 128-K stages): the issuing thread is a serial instruction
                // stream, so every instruction here costs tensor-pipe time.  MMA k of a stage goes to accumulator
                // k % nacc (nacc = 1, 2 or 4); only the first use of an accumulator overwrites it.
                const int nfull = min(nstages, p.KC / 2 - stage0);
                const uint32_t dk1 = tmem_base + (1u % nacc) * NTc, dk2 = tmem_base + (2u % nacc) * NTc,
                               dk3 = tmem_base + (3u % nacc) * NTc;
                const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
                uint32_t f0 = 0, f1 = nacc > 1 ? 0u : 1u, f2 = nacc > 2 ? 0u : 1u, f3 = nacc > 3 ? 0u : 1u;
                for (; i < nfull; ++i, bq.next(), aq.next()) {
                    if (!p.merged && !mbar_wait(&bars[BAR_B_FULL + bq.slot], bq.ph, abort_flag)) { live = false; break; }
                    if (!mbar_wait(&bars[BAR_A_FULL + aq.slot], aq.ph, abort_flag)) { live = false; break; }
                    tc_fence_after();
                    if (mtrace && i < 8) mtrace[8 + i] = trace_now();
                    uint32_t a_addr = tmem_a + aq.slot * 32;
                    uint32_t b_lo = b_lo0 + (uint32_t)bq.slot * b_desc_step;
                    asm volatile(
                        "{\n\t.reg .pred p0, p1, p2, p3;\n\t.reg .b64 d0, d1, d2, d3;\n\t"
                        "setp.ne.b32 p0, %7, 0;\n\t"
                        "setp.ne.b32 p1, %8, 0;\n\t"
                        "setp.ne.b32 p2, %9, 0;\n\t"
                        "setp.ne.b32 p3, %10, 0;\n\t"
                        "mov.b64 d0, {%1, %6};\n\t"
                        "add.u32 %1, %1, 2;\n\t"
                        "mov.b64 d1, {%1, %6};\n\t"
                        "add.u32 %1, %1, 2;\n\t"
                        "mov.b64 d2, {%1, %6};\n\t"
                        "add.u32 %1, %1, 2;\n\t"
                        "mov.b64 d3, {%1, %6};\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%2], [%0], d0, %11, p0;\n\t"
                        "add.u32 %0, %0, 8;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%3], [%0], d1, %11, p1;\n\t"
                        "add.u32 %0, %0, 8;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%4], [%0], d2, %11, p2;\n\t"
                        "add.u32 %0, %0, 8;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%5], [%0], d3, %11, p3;\n\t}"
                        : "+r"(a_addr), "+r"(b_lo)
                        : "r"(tmem_base), "r"(dk1), "r"(dk2), "r"(dk3), "r"(b_hi), "r"(f0), "r"(f1), "r"(f2), "r"(f3), "r"(p.idesc)
                        : "memory");
                    f0 = f1 = f2 = f3 = 1;
                    tc_commit(&bars[BAR_A_EMPTY + aq.slot]);
                    if (!p.merged) tc_commit(&bars[BAR_B_EMPTY + bq.slot]);
                }
                started = f0 ? nacc : 0;
            }
            for (; i < nstages && live; ++i, bq.next(), aq.next()) {
                if (!p.merged && !mbar_wait(&bars[BAR_B_FULL + bq.slot], bq.ph, abort_flag)) break;
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
                if (!p.merged) tc_commit(&bars[BAR_B_EMPTY + bq.slot]);
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
            if (trace && i < 6) trace[16 + i] = trace_now();
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
            // the packed-weight slot goes back only after the stores that consumed the loaded registers have completed: an
            // arrive issued right after the shared-memory loads can be performed while they are still in flight
            mbar_arrive(&bars[BAR_W_EMPTY + ws]);
            tc_fence_before();
            mbar_arrive(&bars[BAR_A_FULL + as]);
            if (trace && i < 6) trace[22 + i] = trace_now();
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
        if (p.ksplit > 1) cluster_wait();                 // barrier #1 (arrived at kernel start): every CTA of the cluster is running
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
                const int per = p.NT / p.ksplit;                  // K split: token columns each CTA of the cluster finishes
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
                    if (p.ksplit == 1) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) stg[(gi * 16 + j) * MMF_TILE_ROWS + row] = (int32_t)v0[j];
                    } else {
                        // straight from registers into the landing zone of the CTA that finishes the column, slot
                        // [my rank] (the own columns included): part[rank][column in the owner's slice][row]
                        int o = (gi * 16) / per, cl = gi * 16 - o * per;
                        uint32_t dst = peer_addr(part + ((int64_t)ks * per) * MMF_TILE_ROWS + row, (uint32_t)o);
                        uint32_t rbar = p.async_red ? peer_addr(&bars[BAR_RED], (uint32_t)o) : 0u;
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (p.async_red) st_async_b32(dst + (uint32_t)(cl * MMF_TILE_ROWS * 4), v0[j], rbar);
                            else st_cluster_b32(dst + (uint32_t)(cl * MMF_TILE_ROWS * 4), v0[j]);
                            if (++cl == per) {
                                cl = 0;
                                if (++o < p.ksplit) {
                                    dst = peer_addr(part + ((int64_t)ks * per) * MMF_TILE_ROWS + row, (uint32_t)o);
                                    if (p.async_red) rbar = peer_addr(&bars[BAR_RED], (uint32_t)o);
                                }
                            }
                        }
                    }
                }
            }
        }
        if (p.ksplit == 1) asm volatile("bar.sync 1, %0;" ::"n"(UNPACK_THREADS) : "memory");   // the 8 epilogue warps only
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
            if (p.async_red) {
                // every partial sum destined for this CTA credits BAR_RED on arrival: wait for this CTA's own bytes only.  A
                // CTA that leaves after this wait has nothing in flight towards it, and its own pushes go to CTAs that stay
                // until they have received them.
                ok = __all_sync(0xffffffffu, mbar_wait(&bars[BAR_RED], 0, abort_flag)) && ok;
            } else {
                cluster_arrive();                             // barrier #2 orders all pushes before the owners' reads
                cluster_wait();
            }
            trace_mark(trace, 6);
            if (ok && !*abort_flag) {
                for (int cl = cth; cl < per; cl += UNPACK_THREADS / 16) {
                    const int c = ks * per + cl;
                    const int m = m0 + c;
                    if (m >= a.M) break;
                    int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                    for (int peer = 0; peer < 8; ++peer) {
                        if (peer < p.ksplit) {
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

    if (p.ksplit > 1 && warp >= NUM_UNPACK_WARPS) {   // the three service warps take part in the cluster barriers
        cluster_wait();
        if (!p.async_red) {
            cluster_arrive();
            cluster_wait();
        }
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

}  // namespace

// Configuration overrides for kernel experiments.  They exist only in the experiments build (-DMMF_EXPERIMENTS, a
// second shared library that the configuration-sweep tests load); the product library has no mutable global state:
// every override is the constant 0 (automatic) there and the code paths it selects are compiled out.
#ifdef MMF_EXPERIMENTS
#include "../../include/mmfree_b200_experiments.h"
static int g_force_ksplit = 0, g_force_nt = 0, g_force_deep = 0, g_force_wt = 0, g_force_sb = 0, g_force_sa = 0, g_force_sw = 0, g_force_persistent = 0, g_force_nacc = 0, g_force_async_red = 0;
extern int g_probe_commits;
extern int g_probe_issuers;
extern int g_pf_skip;

extern "C" int mmf_tuning(int knob, int value) {
    switch (knob) {
        case MMF_TUNE_KSPLIT: g_force_ksplit = value; return MMF_OK;
        case MMF_TUNE_TOKEN_TILE: g_force_nt = value; return MMF_OK;
        case MMF_TUNE_DEEP_RING: g_force_deep = value; return MMF_OK;
        case MMF_TUNE_WEIGHT_TILES: g_force_wt = value; return MMF_OK;
        case MMF_TUNE_B_STAGES: g_force_sb = value; return MMF_OK;
        case MMF_TUNE_A_STAGES: g_force_sa = value; return MMF_OK;
        case MMF_TUNE_W_STAGES: g_force_sw = value; return MMF_OK;
        case MMF_TUNE_PERSISTENT: g_force_persistent = value; return MMF_OK;
        case MMF_TUNE_PROBE_COMMITS: g_probe_commits = value; return MMF_OK;
        case MMF_TUNE_PROBE_ISSUERS: g_probe_issuers = value; return MMF_OK;
        case MMF_TUNE_PREFILL_SKIP: g_pf_skip = value; return MMF_OK;
        case MMF_TUNE_ACCUMULATORS: g_force_nacc = value; return MMF_OK;
        case MMF_TUNE_ASYNC_REDUCE: g_force_async_red = value; return MMF_OK;
        default: return mmf_set_error(MMF_ERR_BAD_ARG, "mmf_tuning: unknown knob %d", knob);
    }
}
#else
static constexpr int g_force_ksplit = 0, g_force_nt = 0, g_force_deep = 0, g_force_wt = 0, g_force_sb = 0, g_force_sa = 0, g_force_sw = 0, g_force_persistent = 0, g_force_nacc = 0, g_force_async_red = 0;
#endif

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
                    // ring depths measured on whole decode steps (batch 32 / 64 / 128): six A / activation stages instead of
                    // four are worth 4 % at 64 token columns and 2.5 % at 128, a 16-deep packed-weight ring (more of the
                    // weight stream fetched while the preceding kernel still runs) another 5 % at 64 columns but -8 % at 128
                    p.SA = p.SB = NT <= 128 ? 6 : 4;
                    p.SW = NT >= 128 ? 8 : NT <= 64 ? 16 : 12;
                    // one accumulator: the issuing thread needs about 67 cycles per MMA, which already exceeds the pipe time of a
                    // dependent small-N MMA, and every extra accumulator is one more TMEM read round trip in the epilogue
                    p.nacc = 1;
                    if (g_force_nacc && g_force_nacc * NT <= 128) p.nacc = g_force_nacc;
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
                p.merged = (mode == 0 && p.SA == p.SB) ? 1 : 0;
                if (smem + 4096 > 227 * 1024) continue;   // the kernel's static shared memory comes on top
                const int64_t ctas = (int64_t)((n_tiles + p.wt - 1) / p.wt) * m_tiles * ks;
                // Latency model in microseconds.  Inside a decode step the kernel starts while its predecessor
                // still runs and fills its rings with weights before the activations exist, so what counts is the
                // path after the dependency wait: fixed set-up / TMA round trip / epilogue, 0.24 us per 128-K stage
                // (0.30 at 256 token columns), and for a K split the cluster barriers and the push reduction.  More
                // split than a stand-alone launch would want wins there (measured on the whole step).  Clusters of
                // 8 with more than 32 token columns no longer fit side by side (measured +6 us).
                const int64_t waves = (ctas + 148 * occ - 1) / (148 * occ);
                const double t_stage = mode == 2 ? 0.90 : NT > 128 ? 0.30 : 0.24;   // (two tiles per CTA measured slower: kept for experiments)
                double t = 2.5 + stages * t_stage + 0.5 + p.wt * NT * 0.012;
                if (ks > 1) t += 0.75 + 0.22 * ks + NT * 0.012 + (ks == 8 && NT > 32 ? 6.0 : 0.0);   // measured: 1.2 / 1.6 / 2.5 us at 2 / 4 / 8
                const double cost = waves * t;
                if (cost < best_cost) { best_cost = cost; best = p; best_smem = smem; found = true; }
            }
        }
    }
    return found;
}

}  // namespace

int bitlinear_mma_launch(const BitLinearArgs& a, cudaStream_t st) {
    {
        // many token rows: the persistent kernel (one CTA per SM) once it has a full wave of work;
        // knob values >= 10 select experimental variant (value - 10) and force it for every M > 128
        const int variant = g_force_persistent >= 10 ? g_force_persistent - 10 : 0;
        const int nt = bitlinear_mma_prefill_tile(a, variant);
        const int64_t n_work = (int64_t)((a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS) * ((a.M + nt - 1) / nt);
        const bool tuned = g_force_ksplit || g_force_nt || g_force_deep || g_force_wt || g_force_sb || g_force_sa || g_force_sw;
        if ((g_force_persistent == 1 || g_force_persistent >= 10) ? a.M > 128
                                                                   : (g_force_persistent == 0 && !tuned && a.M >= 512 && n_work >= 148))
            return bitlinear_mma_prefill_launch(a, st, variant);
    }
    MmaParams p;
    size_t smem = 0;
    MMF_REQUIRE(choose_config(a, p, smem), MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): no kernel configuration fits M=%d N=%d K=%d", a.M,
                a.N, a.K);
    const int m_tiles = (a.M + p.NT - 1) / p.NT;
    p.async_red = g_force_async_red == 1 ? 1 : g_force_async_red == 2 ? 0 : MMF_ASYNC_REDUCE_DEFAULT;
    // instruction descriptor: D=S32, A=S8 (TMEM), B=S8 (smem, K-major), M=128, N=NT
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    MmfEncodeTiledFn encode = mmf_encode_tiled();
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
