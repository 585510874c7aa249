// BitLinear for many token rows (prefill): a persistent tcgen05 kind::i8 kernel, one CTA per SM.
//
// Same operand scheme as the small-batch kernel — 128-row weight tile on the MMA's M axis, its 2-bit
// stream expanded in registers and written straight into tensor memory (A-from-TMEM), int8 activation
// codes fetched by tiled TMA with the 128-byte swizzle — but organised for throughput instead of latency:
//
//  * the single thread that issues the MMAs is a serial instruction stream in which one tcgen05.mma costs
//    about 67 cycles and one tcgen05.commit about 90 (measured), so a stage of four MMAs must not carry
//    more than one commit and one barrier wait: the unpacked-A ring (TMEM) and the activation ring (shared
//    memory) share their barriers — one "full" barrier per stage collects the arrivals of an unpack group
//    plus the TMA transaction bytes, one "empty" barrier (a single commit) hands both buffers back.  The
//    activation ring is eight stages deep on those barriers although tensor memory has room for only four
//    A stages (an activation tile comes from L2 with about a microsecond of latency);
//  * two tile shapes: 192 token columns with TWO accumulators (2 x 192 + 4 x 32 A-stage columns = all 512
//    TMEM columns) — the MMAs of the next work item run while the epilogue drains the previous
//    accumulator; and, for long K, 256 token columns with one accumulator and rings six deep — each MMA
//    then fills the tensor pipe for 133 cycles, which hides the issue cost completely, and the exposed
//    epilogue is amortised over many stages;
//  * pairs of CTAs (a cluster of two, tcgen05 cta_group::2) whenever the weight tiles pair up: each CTA keeps
//    its own weight tile, A ring, accumulators and epilogue, but loads only half of every activation tile;
//    one thread of the even CTA issues 256-row MMAs for both, whose commits reach both CTAs' barriers;
//  * every CTA (pair) walks a list of (weight tile (pair), token tile) work items, weight tile fastest, so that
//    the CTAs running at the same time share a few activation tiles in L2; barriers, TMEM and the three
//    rings (packed weights, unpacked A stages, activation tiles) are set up once and keep streaming
//    across work items — while the epilogue drains one accumulator, the producers and the unpack warps
//    already fill the rings for the next item;
//  * dedicated epilogue warps read the int32 accumulator from TMEM in 16-column chunks, subtract the
//    per-token code sum (weights are stored +1 biased), dequantise and store; the accumulator is handed
//    back to the MMA warp as soon as its last chunk sits in registers.
//
// Warp roles: warp 0 owns tensor memory and issues the MMAs, warps 2 and 3 produce the packed-weight and the
// activation ring, then 4 x GROUPS unpack warps (groups of four take 128-K stages in turn), then 8 epilogue warps
// (TMEM lane quarter = warp % 4, column half by warp).  Every wait is bounded and reports through the status word.
//
// What paces it (measured with parts switched off, timing only): with no activation loads, no weight expansion and
// no output stores the loop reaches 95 % of the tensor pipe with one issuing thread, so the issuing thread is not
// the limit by itself; output stores cost 16 points, activation loads 11, the weight expansion 3.  A stage then
// takes the issuing thread about 480 cycles against 400 of pipe time, with or without a second issuing thread,
// with the issuer in the first or the last warp, and with or without probing the next stage's barrier early.
#include "bitlinear.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {

// Compile-time shape of one variant of the kernel.
template <int NT_, int GROUPS_, int SA_, int SB_, int SW_, bool DOUBLE_, bool MERGED_, bool STAGE_OUT_, int ISSUERS_ = 1, bool PAIR_ = false>
struct PfCfg {
    static constexpr int NT = NT_;                   // token columns per tile
    static constexpr int GROUPS = GROUPS_;           // unpack groups of four warps that take 128-K stages in turn
    static constexpr int SA = SA_;                   // unpacked A stages in TMEM (32 columns each, after the accumulators)
    static constexpr int SB = SB_;                   // activation stages (NT * 128 bytes each)
    static constexpr int SW = SW_;                   // packed-weight stages (4 KB each)
    static constexpr int NACC = DOUBLE_ ? 2 : 1;     // accumulators: with two, MMAs of the next item overlap the epilogue
    // MERGED: the A ring and the activation ring share their barriers: one "full" barrier per stage (128 unpack arrivals +
    // the TMA producer's expect_tx) and one "empty" barrier, so the issuing thread executes one wait and one
    // tcgen05.commit per stage instead of two of each.  The barriers are indexed by the activation ring (depth SB, a
    // multiple of SA): stage s uses activation slot s % SB and A slot s % SA, and the unpack group that refills an A slot
    // waits for the commit of stage s - SA (barrier (s - SA) % SB).  The activation ring can thus run further ahead than
    // the four A stages tensor memory has room for — an activation tile comes from L2 with about a microsecond of latency.
    static constexpr bool MERGED = MERGED_;
    static constexpr int AR = MERGED_ ? SB_ : SA_;   // number of A_FULL / A_EMPTY barriers
    // ISSUERS: threads (one per warp) that issue the MMAs of a stage, each for its own NT / ISSUERS token columns of the
    // tile and of the accumulator.  In a bare issue loop the ~67 cycles an MMA costs its issuing thread overlap between
    // two threads (69 cycles per MMA with one thread, 35 with two).  In this kernel two issuers changed nothing
    // (each still executes four MMAs, a commit and a wait per stage, and it is that per-stage sequence, slowed by the
    // epilogue warps sharing its scheduler, that paces the loop), so the compiled default is one; shapes 5 and 6 keep the
    // two-issuer form for comparison.
    static constexpr int ISSUERS = ISSUERS_;
    static constexpr int NH = NT / ISSUERS;          // token columns per issuer
    static constexpr int UNPACK_WARPS = 4 * GROUPS, EPI_WARPS = 8;
    // warps 0..3: MMA issuer(s), packed-weight producer, activation producer; then the unpack warps, then the epilogue warps
    // (both start at a multiple of four: warp % 4 is the tensor-memory lane quarter a warp may touch)
    static constexpr int WARP_MMA = 0, WARP_W = 2, WARP_B = 3, UNPACK0 = 4, EPI0 = UNPACK0 + UNPACK_WARPS;
    static constexpr int THREADS = (EPI0 + EPI_WARPS) * 32;
    // PAIR: two CTAs (a cluster of two, on two SMs) work as one MMA unit (cta_group::2).  Each owns one weight tile of a
    // pair — its own packed-weight stream, unpack warps, A ring, accumulators and epilogue, exactly as alone — but the
    // activation tile is split: each CTA loads NT / 2 of its token rows, and the MMAs, issued by one thread of the even
    // CTA for both, read both halves.  An activation byte is then written to shared memory once per 256 weight rows
    // instead of once per 128: with the B operand read at 61 bytes per clock by the tensor pipe and written at the same
    // rate by TMA, a single CTA sits at the bandwidth of its shared memory.
    static constexpr bool PAIR = PAIR_;
    static constexpr int CG = PAIR_ ? 2 : 1;
    static constexpr int B_ROWS = PAIR_ ? NT / 2 : NT;   // token rows of the tile this CTA loads
    static constexpr int B_STAGE = B_ROWS * 128;
    static constexpr int W_STAGE = 2 * MMF_TILE_ROWS * 16;
    // STAGE_OUT: 2-byte outputs leave through a shared-memory tile and two TMA stores per work item.  The epilogue warps
    // read the accumulator in the 16x256b fragment layout (a thread holds two adjacent token columns of rows r and r + 8,
    // like an MMA accumulator fragment), convert pairs with one packed instruction and transpose with stmatrix: 2 loads +
    // 2 stmatrix per 16 columns x 32 rows instead of 1 load + 16 two-byte stores.  The tile is two [NT][64 rows] halves in
    // the 128-byte-swizzle layout (stmatrix writes conflict-free; the TMA store undoes the swizzle).
    static constexpr bool STAGE_OUT = STAGE_OUT_;
    static constexpr int OUT_STAGE = STAGE_OUT ? NT * MMF_TILE_ROWS * 2 : 0;
    static constexpr int SMEM = 1024 + SB * B_STAGE + SW * W_STAGE + OUT_STAGE;
    static constexpr int B_FULL = 0, B_EMPTY = B_FULL + SB, W_FULL = B_EMPTY + SB, W_EMPTY = W_FULL + SW,
                         A_FULL = W_EMPTY + SW, A_EMPTY = A_FULL + AR, ACC_FULL = A_EMPTY + AR, ACC_EMPTY = ACC_FULL + 2,
                         BAR_COUNT = ACC_EMPTY + 2;
    static_assert(NACC * NT + SA * 32 <= 512, "accumulators and the A ring must fit tensor memory");
    static_assert(!MERGED || SB % SA == 0, "merged rings: the activation ring is a whole number of A rings deep");
    __host__ __device__ static constexpr int b_full(int slot) { return (MERGED ? A_FULL : B_FULL) + slot; }
    __host__ __device__ static constexpr int b_empty(int slot) { return (MERGED ? A_EMPTY : B_EMPTY) + slot; }
    static_assert(NT % 32 == 0 && NT <= 256, "token tile");
    static_assert((ISSUERS == 1 || ISSUERS == 2) && NH % 16 == 0, "each issuer's columns: a multiple of 16 (MMA N) and of 8 (swizzle atom)");
    static_assert(!PAIR || (MERGED && ISSUERS == 1 && NT % 32 == 0), "pair mode: merged rings, one issuer");
    static_assert(SMEM + 5 * 1024 <= 227 * 1024, "shared memory (dynamic + static) per CTA");
    __device__ static uint32_t bar_count(int i) {
        if (i >= ACC_EMPTY) return (uint32_t)(EPI_WARPS * CG);   // pair: the other CTA's epilogue warps arrive here too
        if (i >= A_EMPTY) return (uint32_t)ISSUERS;              // A_EMPTY, ACC_FULL: one tcgen05.commit per issuer
        // per CTA: one unpack group + the activation producer; in pair mode lane 0 of each unpack warp arrives for its warp
        // (an arrive that crosses to the other CTA costs far more than a local one: 128 of them per stage ran the kernel
        // at 40 % of its speed)
        if (MERGED && i >= A_FULL) return PAIR ? 9u : 129u;   // pair: 2 x 4 unpack warps + the issuing CTA's activation producer
        if (i >= W_EMPTY) return 128u;                           // W_EMPTY, A_FULL: the 128 threads of one unpack group
        if (i >= B_EMPTY && i < W_FULL) return (uint32_t)ISSUERS;
        return 1u;
    }
};

#ifdef MMF_EXPERIMENTS
#define PF_SKIP(x) (x)
#else
#define PF_SKIP(x) false
#endif

struct PfParams {
    int KC;            // K / 64
    int n_tiles;       // weight tiles
    int group_tiles;   // weight tiles per group
    int m_tiles;       // token tiles
    int n_work;        // work items: (weight tile, token tile), in pair mode (pair of weight tiles, token tile)
    int tile_slots;    // weight-tile slots per token tile: n_tiles, in pair mode n_tiles / 2
    int tma_out;       // outputs go through the shared-memory tile and out_map (2-byte dtype, 16-byte aligned rows)
    int skip;          // experiments build only (wrong results, timing only): 1 = no activation loads, 2 = no weight
                       // expansion, 4 = no output stores; 0 in the product build
    uint32_t idesc;
};

struct PfRing {
    int slot, ph, depth;
    __device__ __forceinline__ void next() { if (++slot == depth) { slot = 0; ph ^= 1; } }
};

// One 16-column chunk of the accumulator (this thread: weight row n, token columns c0..c0+15) -> global memory.
template <typename T>
__device__ __forceinline__ void pf_store_chunk(const BitLinearArgs& a, const uint32_t (&v)[16], const int* rs, const float* sc,
                                               int m, int n, int ncols) {
    T* p = reinterpret_cast<T*>(a.out) + (int64_t)m * a.ld_out + n;
    if (ncols >= 16) {
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            const int4 r4 = *reinterpret_cast<const int4*>(rs + j4 * 4);
            const float4 s4 = *reinterpret_cast<const float4*>(sc + j4 * 4);
            const int rr[4] = {r4.x, r4.y, r4.z, r4.w};
            const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                *p = from_f32<T>(__fmul_rn((float)((int32_t)v[j4 * 4 + j] - rr[j]), ss[j]));
                p += a.ld_out;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (j < ncols) *p = from_f32<T>(__fmul_rn((float)((int32_t)v[j] - rs[j]), sc[j]));
            p += a.ld_out;
        }
    }
}

// accumulator fragment: 16 TMEM lanes x 16 columns starting at `taddr`; thread t receives, for the two 8-column blocks
// k = 0, 1: r[4k] = (lane t/4, column 8k + 2(t%4)), r[4k+1] = (same lane, next column), r[4k+2], r[4k+3] = lane t/4 + 8
__device__ __forceinline__ void tmem_ld_frag16(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// four 8x8 matrices of 16-bit elements, each stored transposed: thread 8i + j supplies the address of the 16 bytes that
// receive column j of matrix i
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t smem_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(smem_addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}
__device__ __forceinline__ uint32_t pack_out2(float lo, float hi, int out_dtype) {
    if (out_dtype == MMF_BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <typename C>
__global__ void __launch_bounds__(C::THREADS, 1)
bitlinear_mma_prefill_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap out_map,
                             BitLinearArgs a, PfParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* b_ring = base;
    uint8_t* w_ring = base + C::SB * C::B_STAGE;

    __shared__ __align__(8) uint64_t bars[C::BAR_COUNT];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ __align__(16) float s_scale[2][C::NT];   // dq[m] * w_scale per token column, double-buffered by work item
    __shared__ __align__(16) int s_rs[2][C::NT];        // code sum per token column

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    pdl_trigger();
    if (threadIdx.x == 0) { tma_prefetch_map(&q_map); tma_prefetch_map(&out_map); }

    if (tid < C::BAR_COUNT) mbar_init(&bars[tid], C::bar_count(tid));
    if (tid == C::BAR_COUNT) s_abort = 0;
    if (warp == C::WARP_MMA) tmem_alloc_cg<C::CG>(&s_tmem_base, 512u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (C::PAIR) { cluster_arrive(); cluster_wait(); }   // the other CTA's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t rank = C::PAIR ? cluster_ctarank() : 0u;   // 0: the CTA that issues the pair's MMAs
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t tmem_a = tmem_base + C::NACC * C::NT;
    volatile int* abort_flag = &s_abort;
    const int S = (p.KC + 1) / 2;              // 128-K stages per work item
    const int first = C::PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x, step = C::PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    // work item -> this CTA's weight tile (pair mode: tiles 2s and 2s + 1 of slot s) and the token tile
    auto item_tile = [&](int wk) { return C::PAIR ? 2 * (wk % p.tile_slots) + (int)rank : wk % p.tile_slots; };
    // optional phase trace of CTA 0 (armed by MMF_TRACE_MAGIC in workspace word 1): 28 clock64 slots in the header
    long long* trace = MMF_TRACE_PTR((lane == 0 && blockIdx.x == 0 && a.ws && a.ws[1] == MMF_TRACE_MAGIC)
                           ? reinterpret_cast<long long*>(a.ws + 8) : nullptr);
    if (tid == 0) { trace_mark(trace, 0); if (trace) trace[26] = clock64(); }   // 26 / 27: SM clock count at both ends

    if (warp == C::WARP_W) {
        // ------------------------------------------------------------ packed weights (bulk TMA); independent of the
        // preceding kernel, so the stream starts before the grid dependency wait
        if (elect_one()) {
            PfRing w{0, 0, C::SW};
            bool live = true;
            for (int wk = first; wk < p.n_work && live; wk += step) {
                const int tile = item_tile(wk);
                const uint8_t* src = reinterpret_cast<const uint8_t*>(a.packed) + (int64_t)tile * p.KC * (MMF_TILE_ROWS * 16);
                for (int i = 0; i < S; ++i, w.next()) {
                    const uint32_t bytes = (uint32_t)min(2, p.KC - i * 2) * (MMF_TILE_ROWS * 16);
                    if (!mbar_wait(&bars[C::W_EMPTY + w.slot], w.ph ^ 1, abort_flag)) { live = false; break; }
                    mbar_expect_tx(&bars[C::W_FULL + w.slot], bytes);
                    bulk_load_1d(w_ring + w.slot * C::W_STAGE, src + (int64_t)i * C::W_STAGE, bytes, &bars[C::W_FULL + w.slot]);
                }
            }
        }
    } else if (warp == C::WARP_B) {
        // ------------------------------------------------------------ activation tiles (TMA, 128-byte swizzle)
        pdl_wait();
        if (elect_one()) {
            PfRing bq{0, 0, C::SB};
            bool live = true;
            for (int wk = first; wk < p.n_work && live; wk += step) {
                const int tile = item_tile(wk), mt = wk / p.tile_slots;
                const int y = (tile / p.group_tiles) * a.M + mt * C::NT + (int)rank * C::B_ROWS;
                for (int i = 0; i < S; ++i, bq.next()) {
                    if (!mbar_wait(&bars[C::b_empty(bq.slot)], bq.ph ^ 1, abort_flag)) { live = false; break; }
                    if (C::PAIR && rank != 0) {
                        if (PF_SKIP(p.skip & 1)) continue;
                        // this CTA's half of the tile lands here; its bytes are counted by the issuing CTA's "full" barrier,
                        // whose own producer announces the bytes of both halves (a transaction count may run negative)
                        tma_load_2d_pair(b_ring + bq.slot * C::B_STAGE, &q_map, cluster_addr(&bars[C::b_full(bq.slot)], 0u), i * 128, y);
                        continue;
                    }
                    if (PF_SKIP(p.skip & 1)) { mbar_arrive(&bars[C::b_full(bq.slot)]); continue; }
                    mbar_expect_tx(&bars[C::b_full(bq.slot)], (uint32_t)(C::CG * C::B_STAGE));
                    tma_load_2d(b_ring + bq.slot * C::B_STAGE, &q_map, &bars[C::b_full(bq.slot)], i * 128, y);
                }
            }
        }
    } else if (warp < C::ISSUERS) {
        // ------------------------------------------------------------ MMA issue: a serial instruction stream per issuer,
        // kept short; issuer `half` owns token columns [half * NH, half * NH + NH) of the tile and of the accumulator
        if (elect_one() && rank == 0) {
            const int half = warp - C::WARP_MMA;
            if (half != 0) trace = nullptr;
            PfRing bq{0, 0, C::SB}, aq{0, 0, C::SA};
            const uint64_t b_desc0 = make_b_desc(smem_u32(b_ring + half * (C::NH * 128)));
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            const uint32_t b_desc_step = (uint32_t)C::B_STAGE >> 4;
            const int nfull = p.KC / 2;          // whole 128-K stages; a trailing 64-K stage issues two MMAs
            bool live = true;
            int it = 0;
            for (int wk = first; wk < p.n_work && live; wk += step, ++it) {
                // the epilogue must have drained this accumulator (used two work items ago)
                const int ab = C::NACC == 2 ? (it & 1) : 0;              // accumulator of this work item
                if (!mbar_wait(&bars[C::ACC_EMPTY + ab], (uint32_t)(((it / C::NACC) & 1) ^ 1), abort_flag)) break;
                tc_fence_after();
                const uint32_t d_addr = tmem_base + (uint32_t)ab * C::NT + (uint32_t)half * C::NH;
                if (it >= 1 && it < 5) trace_mark(trace, 1 + (it - 1) * 3);
                
                uint32_t accum = 0;
                for (int i = 0; i < S; ++i, bq.next(), aq.next()) {
                    if (!mbar_wait(&bars[C::b_full(bq.slot)], bq.ph, abort_flag)) { live = false; break; }
                    if (!C::MERGED && !mbar_wait(&bars[C::A_FULL + aq.slot], aq.ph, abort_flag)) { live = false; break; }
                    tc_fence_after();
                    if (i == 0 && it >= 1 && it < 5) trace_mark(trace, 2 + (it - 1) * 3);
                    uint32_t a_addr = tmem_a + aq.slot * 32;
                    uint32_t b_lo = b_lo0 + (uint32_t)bq.slot * b_desc_step;
                    if (i < nfull) {
#define PF_FOUR_MMAS(CGS)                                                                                        \
                        asm volatile(                                                                            \
                            "{\n\t.reg .pred p;\n\t.reg .b64 d0, d1, d2, d3;\n\t"                                 \
                            "setp.ne.b32 p, %4, 0;\n\t"                                                          \
                            "mov.b64 d0, {%1, %3};\n\t"                                                          \
                            "add.u32 %1, %1, 2;\n\t"                                                             \
                            "mov.b64 d1, {%1, %3};\n\t"                                                          \
                            "add.u32 %1, %1, 2;\n\t"                                                             \
                            "mov.b64 d2, {%1, %3};\n\t"                                                          \
                            "add.u32 %1, %1, 2;\n\t"                                                             \
                            "mov.b64 d3, {%1, %3};\n\t"                                                          \
                            "tcgen05.mma.cta_group::" CGS ".kind::i8 [%2], [%0], d0, %5, p;\n\t"                  \
                            "add.u32 %0, %0, 8;\n\t"                                                             \
                            "tcgen05.mma.cta_group::" CGS ".kind::i8 [%2], [%0], d1, %5, 1;\n\t"                  \
                            "add.u32 %0, %0, 8;\n\t"                                                             \
                            "tcgen05.mma.cta_group::" CGS ".kind::i8 [%2], [%0], d2, %5, 1;\n\t"                  \
                            "add.u32 %0, %0, 8;\n\t"                                                             \
                            "tcgen05.mma.cta_group::" CGS ".kind::i8 [%2], [%0], d3, %5, 1;\n\t}"                 \
                            : "+r"(a_addr), "+r"(b_lo)                                                           \
                            : "r"(d_addr), "r"(b_hi), "r"(accum), "r"(p.idesc)                                   \
                            : "memory")
                        if constexpr (C::PAIR) PF_FOUR_MMAS("2"); else PF_FOUR_MMAS("1");
#undef PF_FOUR_MMAS
                    } else {
                        const uint64_t bd = ((uint64_t)b_hi << 32) | b_lo;
                        mma_i8_ts_cg<C::CG>(d_addr, a_addr, bd, p.idesc, accum);
                        mma_i8_ts_cg<C::CG>(d_addr, a_addr + 8, bd + 2, p.idesc, 1u);
                    }
                    accum = 1;
                    tc_commit_cg<C::CG>(&bars[C::b_empty(bq.slot)]);   // frees the activation stage (merged: and the A stage; pair: in both CTAs) when these MMAs retire
                    if (!C::MERGED) tc_commit(&bars[C::A_EMPTY + aq.slot]);
                }
                if (live) tc_commit_cg<C::CG>(&bars[C::ACC_FULL + ab]);
                if (it >= 1 && it < 5) trace_mark(trace, 3 + (it - 1) * 3);
            }
            trace_mark(trace, 25);
            if (trace) trace[27] = clock64();
        }
    } else if (warp < C::UNPACK0) {
        // spare warp of the first four
    } else if (warp < C::EPI0) {
        // ------------------------------------------------------------ unpack: lane <-> TMEM lane <-> weight row
        const int qd = warp & 3, gp = (warp - C::UNPACK0) >> 2;
        const int row = qd * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
        PfRing w{0, 0, C::SW}, aq{0, 0, C::SA};
        for (int k = 0; k < gp; ++k) { w.next(); aq.next(); }
        int sg = gp;            // next global stage (counted across work items) this group expands
        int tile_base = 0;      // global index of the current work item's first stage
        bool ok = true;
        for (int wk = first; wk < p.n_work && ok; wk += step, tile_base += S) {
            for (; sg < tile_base + S; sg += C::GROUPS) {
                const int i = sg - tile_base;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars[C::W_FULL + w.slot], w.ph, abort_flag));   // warp-uniform
                if (!ok) break;
                const int nch = min(2, p.KC - i * 2);
                const uint8_t* wsrc = w_ring + w.slot * C::W_STAGE + row * 16;
                uint4 wv[2];
                wv[0] = *reinterpret_cast<const uint4*>(wsrc);
                wv[1] = nch > 1 ? *reinterpret_cast<const uint4*>(wsrc + MMF_TILE_ROWS * 16) : wv[0];
                // the MMAs that read this A slot last (stage sg - SA) must have retired
                if (C::MERGED) {
                    const int t = sg - C::SA;
                    if (t >= 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars[C::A_EMPTY + t % C::SB], (uint32_t)((t / C::SB) & 1), abort_flag));
                } else {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars[C::A_EMPTY + aq.slot], aq.ph ^ 1, abort_flag));
                }
                if (!ok) break;   // uniform per warp: the .sync.aligned tcgen05 ops below need the whole warp
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < nch && !PF_SKIP(p.skip & 2)) {
                        const uint32_t words[4] = {wv[h].x, wv[h].y, wv[h].z, wv[h].w};
                        uint32_t r[16];
#pragma unroll
                        for (int w4 = 0; w4 < 4; ++w4)
#pragma unroll
                            for (int k4 = 0; k4 < 4; ++k4) r[w4 * 4 + k4] = (words[w4] >> (2 * k4)) & 0x03030303u;
                        tmem_st16(tmem_a + lane_addr + aq.slot * 32 + h * 16, r);
                    }
                }
                tmem_wait_st();
                // The packed-weight slot goes back only now, after the stores that consumed the loaded registers have
                // completed.  An arrive placed right after the two shared-memory loads can be performed while those loads
                // are still in flight (nothing orders an mbarrier arrive behind an earlier load whose result it does not
                // use): with a shallow weight ring the refill then overwrote the slot under the second load, and single
                // 8-lane wavefronts of it returned the next work item's weights.
                mbar_arrive(&bars[C::W_EMPTY + w.slot]);
                tc_fence_before();
                if (C::PAIR) {
                    __syncwarp();          // tcgen05.wait::st is warp-wide: every lane's stores have completed
                    if (lane == 0) {
                        if (rank != 0) mbar_arrive_remote(cluster_addr(&bars[C::A_FULL + sg % C::SB], 0u));
                        else mbar_arrive(&bars[C::A_FULL + sg % C::SB]);
                    }
                } else {
                    mbar_arrive(&bars[C::A_FULL + (C::MERGED ? sg % C::SB : aq.slot)]);
                }
#pragma unroll
                for (int k = 0; k < C::GROUPS; ++k) { w.next(); aq.next(); }
            }
            
        }
    } else {
        // ------------------------------------------------------------ epilogue: TMEM -> registers -> global memory
        const int ew = warp - C::EPI0;
        const int lq = ew & 3, hf = ew >> 2;
        const uint32_t lane_addr = (uint32_t)(lq * 32) << 16;
        const int col0 = hf * (C::NT / 2);
        const int eidx = ew * 32 + lane;              // the token column (< NT) whose constants this thread stages
        uint16_t* ostage = reinterpret_cast<uint16_t*>(w_ring + C::SW * C::W_STAGE);   // [NT][128] output tile (STAGE_OUT)
        const bool staged = C::STAGE_OUT && p.tma_out;
        // stmatrix address of this lane for accumulator fragments of lanes [lq*32 + 16*h2, +16): lane 8i + j writes token
        // column 8(i/2) + j of the chunk, rows 8(i%2).. of the fragment; half tile by row / 64, 16-byte chunk XOR (token % 8)
        uint32_t st_off[2];
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            const int i = lane >> 3, j = lane & 7;
            const int n0 = lq * 32 + 16 * h2 + 8 * (i & 1);
            st_off[h2] = (uint32_t)((n0 >> 6) * (C::NT * 128) + (8 * (i >> 1) + j) * 128 + ((((n0 & 63) >> 3) ^ j) << 4));
        }
        const uint32_t ostage_u32 = smem_u32(ostage);
        pdl_wait();                                   // dq / rowsum come from the preceding kernel
        bool ok = true;
        int it = 0;
        for (int wk = first; wk < p.n_work && ok; wk += step, ++it) {
            const int tile = item_tile(wk), mt = wk / p.tile_slots;
            const int g = tile / p.group_tiles;
            const int m0 = mt * C::NT;
            float* sc = s_scale[it & 1];
            int* rs = s_rs[it & 1];
            if (eidx < C::NT) {
                const int m = m0 + eidx;
                const bool in = m < a.M;
                sc[eidx] = in ? __fmul_rn(a.dq[(int64_t)g * a.M + m], a.w_scale[g]) : 0.0f;
                rs[eidx] = in ? a.rowsum[(int64_t)g * a.M + m] : 0;
            }
            // the TMA store of the previous work item must have read the output tile before it is overwritten
            if (staged && ew == 0 && lane == 0) bulk_wait_read<0>();
            asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");   // the 8 epilogue warps only
            const int ab = C::NACC == 2 ? (it & 1) : 0;
            ok = mbar_wait_warp<true>(&bars[C::ACC_FULL + ab], (uint32_t)((it / C::NACC) & 1), abort_flag);
            if (!ok) break;
            tc_fence_after();
            if (ew == 0 && it < 4) trace_mark(trace, 13 + it * 3);
            const int n = tile * MMF_TILE_ROWS + lq * 32 + lane;
            const bool n_ok = n < a.N;
            const int mvalid = min(C::NT / 2, a.M - m0 - col0);    // valid token columns in this warp's half (may be <= 0)
            if (staged) {
                // columns past M carry zero constants and rows past N garbage: the TMA store clips both
                uint32_t fr[2][2][8];
                const uint32_t acc_col = tmem_base + (uint32_t)ab * C::NT + (uint32_t)col0;
                const uint32_t lane_lo = (uint32_t)(lq * 32) << 16, lane_hi = (uint32_t)(lq * 32 + 16) << 16;
                tmem_ld_frag16(acc_col + lane_lo, fr[0][0]);
                tmem_ld_frag16(acc_col + lane_hi, fr[0][1]);
#pragma unroll
                for (int c = 0; c < C::NT / 32; ++c) {
                    tmem_wait_ld();
                    if (c + 1 < C::NT / 32) {
                        tmem_ld_frag16(acc_col + lane_lo + (c + 1) * 16, fr[(c + 1) & 1][0]);
                        tmem_ld_frag16(acc_col + lane_hi + (c + 1) * 16, fr[(c + 1) & 1][1]);
                    } else {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (C::PAIR && rank != 0) mbar_arrive_remote(cluster_addr(&bars[C::ACC_EMPTY + ab], 0u));
                            else mbar_arrive(&bars[C::ACC_EMPTY + ab]);
                        }
                        if (ew == 0 && it < 4) trace_mark(trace, 14 + it * 3);
                    }
                    if (PF_SKIP(p.skip & 4)) continue;
                    const int cc = col0 + c * 16;
                    // this thread's token columns: cc + 8k + 2(lane % 4) and the next one, k = 0, 1
                    const int2 r0 = *reinterpret_cast<const int2*>(rs + cc + 2 * (lane & 3));
                    const int2 r1 = *reinterpret_cast<const int2*>(rs + cc + 8 + 2 * (lane & 3));
                    const float2 s0 = *reinterpret_cast<const float2*>(sc + cc + 2 * (lane & 3));
                    const float2 s1 = *reinterpret_cast<const float2*>(sc + cc + 8 + 2 * (lane & 3));
#pragma unroll
                    for (int h2 = 0; h2 < 2; ++h2) {
                        const uint32_t (&f)[8] = fr[c & 1][h2];
                        const uint32_t p0 = pack_out2(__fmul_rn((float)((int32_t)f[0] - r0.x), s0.x), __fmul_rn((float)((int32_t)f[1] - r0.y), s0.y), a.out_dtype);
                        const uint32_t p1 = pack_out2(__fmul_rn((float)((int32_t)f[2] - r0.x), s0.x), __fmul_rn((float)((int32_t)f[3] - r0.y), s0.y), a.out_dtype);
                        const uint32_t p2 = pack_out2(__fmul_rn((float)((int32_t)f[4] - r1.x), s1.x), __fmul_rn((float)((int32_t)f[5] - r1.y), s1.y), a.out_dtype);
                        const uint32_t p3 = pack_out2(__fmul_rn((float)((int32_t)f[6] - r1.x), s1.x), __fmul_rn((float)((int32_t)f[7] - r1.y), s1.y), a.out_dtype);
                        stmatrix_x4_trans(ostage_u32 + st_off[h2] + (uint32_t)(cc * 128), p0, p1, p2, p3);
                    }
                }
            } else {
            uint32_t v[2][16];
            const uint32_t acc_addr = tmem_base + (uint32_t)ab * C::NT + lane_addr + col0;
            tmem_ld16(acc_addr, v[0]);
#pragma unroll
            for (int c = 0; c < C::NT / 32; ++c) {
                tmem_wait_ld();
                if (c + 1 < C::NT / 32) {
                    tmem_ld16(acc_addr + (c + 1) * 16, v[(c + 1) & 1]);
                } else {
                    // the whole accumulator half is in registers: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (C::PAIR && rank != 0) mbar_arrive_remote(cluster_addr(&bars[C::ACC_EMPTY + ab], 0u));
                        else mbar_arrive(&bars[C::ACC_EMPTY + ab]);
                    }
                    if (ew == 0 && it < 4) trace_mark(trace, 14 + it * 3);
                }
                const int ncols = PF_SKIP(p.skip & 4) ? 0 : mvalid - c * 16;
                if (n_ok && ncols > 0) {
                    const int cc = col0 + c * 16;
                    if (a.acc_out) {
                        for (int j = 0; j < 16 && j < ncols; ++j)
                            a.acc_out[(int64_t)(m0 + cc + j) * a.N + n] = (int32_t)v[c & 1][j] - rs[cc + j];
                    }
                    if (a.out_dtype == MMF_BF16) pf_store_chunk<__nv_bfloat16>(a, v[c & 1], rs + cc, sc + cc, m0 + cc, n, ncols);
                    else if (a.out_dtype == MMF_F16) pf_store_chunk<__half>(a, v[c & 1], rs + cc, sc + cc, m0 + cc, n, ncols);
                    else pf_store_chunk<float>(a, v[c & 1], rs + cc, sc + cc, m0 + cc, n, ncols);
                }
            }
            }
            if (ew == 0 && it < 4) trace_mark(trace, 15 + it * 3);
            if (staged) {
                fence_async_smem();
                asm volatile("bar.sync 1, %0;" ::"n"(C::EPI_WARPS * 32) : "memory");
                if (ew == 0 && lane == 0 && !PF_SKIP(p.skip & 4)) {
                    tma_store_2d(&out_map, ostage, tile * MMF_TILE_ROWS, m0);
                    tma_store_2d(&out_map, reinterpret_cast<const uint8_t*>(ostage) + C::NT * 128, tile * MMF_TILE_ROWS + 64, m0);
                    bulk_commit();
                }
            }
        }
        if (staged && ew == 0 && lane == 0) bulk_wait_all();   // shared memory must outlive the last store
    }

    // teardown: everyone meets, TMEM goes back; on the error path give copies in flight time to land first
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
    tc_fence_before();
    __syncthreads();
    // pair: neither CTA leaves (or frees tensor memory) while the other may still arrive on its barriers, read its half of
    // an activation tile or run MMAs on its tensor memory
    if (C::PAIR) { cluster_arrive(); cluster_wait(); }
    if (warp == C::WARP_MMA) tmem_dealloc_cg<C::CG>(tmem_base, 512u);
}

}  // namespace
#ifdef MMF_EXPERIMENTS
int g_pf_skip = 0;     // mmf_tuning(MMF_TUNE_PREFILL_SKIP, bits)
#else
static constexpr int g_pf_skip = 0;
#endif
namespace {

template <typename C>
int pf_launch(const BitLinearArgs& a, cudaStream_t st) {
    PfParams p;
    p.KC = a.K / MMF_TILE_K;
    p.n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    p.group_tiles = p.n_tiles / a.groups;
    p.m_tiles = (a.M + C::NT - 1) / C::NT;
    p.tile_slots = C::PAIR ? p.n_tiles / 2 : p.n_tiles;
    MMF_REQUIRE(!C::PAIR || (p.n_tiles % 2 == 0 && p.group_tiles % 2 == 0 && a.N % MMF_TILE_ROWS == 0), MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear(mma): the paired kernel needs an even number of whole weight tiles per projection");
    const int64_t n_work = (int64_t)p.tile_slots * p.m_tiles;
    MMF_REQUIRE(n_work < (1ll << 31), MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): problem too large");
    p.n_work = (int)n_work;
    p.skip = g_pf_skip;
    // instruction descriptor: D=S32, A=S8 (TMEM), B=S8 (smem, K-major), M=128 (256 across a pair), N=NH (one issuer's columns)
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(C::NH >> 3) << 17) | ((uint32_t)((C::PAIR ? 256 : 128) >> 4) << 24);

    MmfEncodeTiledFn encode = mmf_encode_tiled();
    MMF_REQUIRE(encode != nullptr, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap q_map;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.groups * (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.K};
    const cuuint32_t box[2] = {128u, (cuuint32_t)C::B_ROWS};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult cr = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(a.q), gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MMF_REQUIRE(cr == CUDA_SUCCESS, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled failed (%d)", (int)cr);

    // output map for the staged epilogue: [M][N] rows of ld_out elements, box = one [NT tokens x 128 rows] tile
    CUtensorMap out_map = q_map;
    p.tma_out = 0;
    // (calls that also want the int32 accumulators take the direct-store epilogue)
    if (C::STAGE_OUT && a.out_dtype != MMF_F32 && !a.acc_out && mmf_aligned(a.out, 16) && (a.ld_out * 2) % 16 == 0) {
        const cuuint64_t odim[2] = {(cuuint64_t)a.N, (cuuint64_t)a.M};
        const cuuint64_t ostride[1] = {(cuuint64_t)a.ld_out * 2};
        const cuuint32_t obox[2] = {64u, (cuuint32_t)C::NT};     // one half tile: [NT tokens][64 rows], 128-byte swizzle
        const CUresult cr2 = encode(&out_map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a.out, odim, ostride, obox, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MMF_REQUIRE(cr2 == CUDA_SUCCESS, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled (output) failed (%d)", (int)cr2);
        p.tma_out = 1;
    }

    int dev = 0, sms = 0;
    MMF_CUDA(cudaGetDevice(&dev));
    MMF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    auto kernel = bitlinear_mma_prefill_kernel<C>;
    MMF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
    cudaLaunchConfig_t cfg = {};
    // one CTA per SM; in pair mode one cluster of two per work item in flight, an even number of CTAs
    const int ctas = C::PAIR ? 2 * (p.n_work < sms / 2 ? p.n_work : sms / 2) : (p.n_work < sms ? p.n_work : sms);
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (C::PAIR) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    MMF_CUDA(cudaLaunchKernelEx(&cfg, kernel, q_map, out_map, a, p));
    MMF_LAUNCH_CHECK("bitlinear_mma_prefill_kernel");
    return MMF_OK;
}

// Compiled shapes.  1: long K — 256-token tile, one accumulator, rings six deep (the main loop is bound by the tensor
// pipe and the exposed epilogue is amortised over many stages).  2: 192-token tile, two accumulators, rings four deep
// (the epilogue of one work item overlaps the main loop of the next).  3: as 2 with the TMA-store epilogue.  4: as 1
// with separate A / activation rings (two waits and two commits per stage), kept for comparison.
using PfLongK = PfCfg<256, 2, 6, 6, 6, false, true, false>;
using PfOverlap = PfCfg<192, 3, 4, 8, 6, true, true, false>;
using PfOverlapTma = PfCfg<192, 3, 4, 4, 8, true, true, true>;
using PfSeparate = PfCfg<256, 2, 8, 5, 8, false, false, false>;
// 5, 6: shapes 1 and 2 with two issuing threads (128 / 96 columns per MMA each), kept for comparison
using PfLongK2 = PfCfg<256, 2, 6, 6, 6, false, true, false, 2>;
using PfOverlap2 = PfCfg<192, 3, 4, 4, 8, true, true, false, 2>;
// 7: shape 2 with the activation ring as deep as the A ring (four stages), as it was before; kept for comparison
using PfOverlapShallow = PfCfg<192, 3, 4, 4, 8, true, true, false>;
// 8, 9: shapes 2 and 1 run by pairs of CTAs (cta_group::2): each CTA loads half of every activation tile
using PfOverlapPair = PfCfg<192, 3, 4, 8, 6, true, true, false, 1, true>;
using PfLongKPair = PfCfg<256, 2, 6, 6, 6, false, true, false, 1, true>;
// 10, 11: shapes 8 and 9 with the stmatrix + TMA-store epilogue
using PfOverlapPairSt = PfCfg<192, 3, 4, 8, 6, true, true, true, 1, true>;
using PfLongKPairSt = PfCfg<256, 2, 6, 6, 6, false, true, true, 1, true>;
// 12: shape 11 with rings eight deep (all of tensor memory: 256 accumulator columns + 8 x 32 A-stage columns)
using PfLongKPairSt8 = PfCfg<256, 2, 8, 8, 6, false, true, true, 1, true>;

// Default: the paired shapes when every projection is a whole, even number of weight tiles (each pair of CTAs then takes
// two tiles of one projection), else the single-CTA shapes.
int pf_pick(const BitLinearArgs& a, int variant) {
    if (variant) return variant;
    const int n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const bool pairs = a.N % MMF_TILE_ROWS == 0 && n_tiles % a.groups == 0 && (n_tiles / a.groups) % 2 == 0;
    if (!pairs) return a.K >= 4096 ? 1 : 2;
    // paired shapes with the stmatrix + TMA-store epilogue: the 256-token tile for long K, and for shorter K when its work
    // items fill the 74 CTA pairs' last round clearly better than those of the 192-token tile (e.g. N = 2048, M = 16384:
    // 512 items = 6.9 rounds against 688 items = 9.3 rounds)
    if (a.K >= 4096) return 12;
    auto fill = [&](int nt) {
        const double items = (double)(n_tiles / 2) * (double)((a.M + nt - 1) / nt), units = 74.0;
        const double rounds = (double)(long long)((items + units - 1) / units);
        return items / (rounds * units);
    };
    return fill(256) > fill(192) + 0.03 ? 12 : 10;
}

}  // namespace

int bitlinear_mma_prefill_tile(const BitLinearArgs& a, int variant) {
    const int v = pf_pick(a, variant);
    return v == 2 || v == 3 || v == 6 || v == 7 || v == 8 || v == 10 ? 192 : 256;
}

// Launch the persistent kernel (large M).  Same argument contract as bitlinear_mma_launch; `variant` selects one
// of the compiled shapes (0 = by problem shape).
int bitlinear_mma_prefill_launch(const BitLinearArgs& a, cudaStream_t st, int variant) {
    switch (pf_pick(a, variant)) {
        case 1: return pf_launch<PfLongK>(a, st);
        case 3: return pf_launch<PfOverlapTma>(a, st);
        case 4: return pf_launch<PfSeparate>(a, st);
        case 5: return pf_launch<PfLongK2>(a, st);
        case 6: return pf_launch<PfOverlap2>(a, st);
        case 7: return pf_launch<PfOverlapShallow>(a, st);
        case 8: return pf_launch<PfOverlapPair>(a, st);
        case 9: return pf_launch<PfLongKPair>(a, st);
        case 10: return pf_launch<PfOverlapPairSt>(a, st);
        case 11: return pf_launch<PfLongKPairSt>(a, st);
        case 12: return pf_launch<PfLongKPairSt8>(a, st);
        default: return pf_launch<PfOverlap>(a, st);
    }
}
