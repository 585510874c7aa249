// BitLinear for many token rows (prefill): a persistent tcgen05 kind::i8 kernel, one CTA per SM.
//
// Same operand scheme as the small-batch kernel — 128-row weight tile on the MMA's M axis, its 2-bit
// stream expanded in registers and written straight into tensor memory (A-from-TMEM), int8 activation
// codes fetched by tiled TMA with the 128-byte swizzle — but organised for throughput instead of latency:
//
//  * 256 token columns per tile: one MMA then occupies the tensor pipe for its full 130 cycles, which
//    also gives the single issuing thread the largest budget per instruction;
//  * every CTA walks a list of (weight tile, token tile) work items, weight tile fastest, so that the
//    CTAs running at the same time share a few activation tiles in L2; barriers, TMEM and the three
//    rings (packed weights, unpacked A stages, activation tiles) are set up once and keep streaming
//    across work items — while the epilogue drains one accumulator, the producers and the unpack warps
//    already fill the rings for the next item;
//  * dedicated epilogue warps read the int32 accumulator from TMEM in 16-column chunks, subtract the
//    per-token code sum (weights are stored +1 biased), dequantise and store; the accumulator is handed
//    back to the MMA warp as soon as its last chunk sits in registers.
//
// Warp roles (608 threads): 0-7 unpack (two groups of four that alternate 128-K stages), 8-15 epilogue
// (TMEM lane quarter = warp % 4, column half = (warp - 8) / 4), 16 packed-weight producer, 17 activation
// producer, 18 TMEM owner + MMA issuer.  Every wait is bounded and reports through the status word.
#include "bitlinear.cuh"
#include "tcgen05.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int PF_NT = 256;                 // token columns per tile
constexpr int PF_UNPACK_WARPS = 8, PF_EPI_WARPS = 8;
constexpr int PF_WARP_W = 16, PF_WARP_B = 17, PF_WARP_MMA = 18;
constexpr int PF_THREADS = 19 * 32;
constexpr int PF_SA = 8;                   // unpacked A stages in TMEM (32 columns each, after the 256 accumulator columns)
constexpr int PF_SB = 5;                   // activation stages (32 KB each)
constexpr int PF_SW = 8;                   // packed-weight stages (4 KB each)
constexpr int PF_B_STAGE = PF_NT * 128;
constexpr int PF_W_STAGE = 2 * MMF_TILE_ROWS * 16;
constexpr int PF_SMEM = 1024 + PF_SB * PF_B_STAGE + PF_SW * PF_W_STAGE;

constexpr int PB_B_FULL = 0, PB_B_EMPTY = PB_B_FULL + PF_SB, PB_W_FULL = PB_B_EMPTY + PF_SB, PB_W_EMPTY = PB_W_FULL + PF_SW,
              PB_A_FULL = PB_W_EMPTY + PF_SW, PB_A_EMPTY = PB_A_FULL + PF_SA, PB_ACC_FULL = PB_A_EMPTY + PF_SA,
              PB_ACC_EMPTY = PB_ACC_FULL + 1, PB_COUNT = PB_ACC_EMPTY + 1;

__device__ __forceinline__ uint32_t pf_bar_count(int i) {
    if (i >= PB_W_EMPTY && i < PB_A_EMPTY) return 128u;   // the 128 threads of one unpack group
    if (i == PB_ACC_EMPTY) return (uint32_t)PF_EPI_WARPS;
    return 1u;
}

struct PfParams {
    int KC;            // K / 64
    int n_tiles;       // weight tiles
    int group_tiles;   // weight tiles per group
    int m_tiles;       // token tiles
    int n_work;        // n_tiles * m_tiles
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

__global__ void __launch_bounds__(PF_THREADS, 1)
bitlinear_mma_prefill_kernel(const __grid_constant__ CUtensorMap q_map, BitLinearArgs a, PfParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* b_ring = base;
    uint8_t* w_ring = base + PF_SB * PF_B_STAGE;

    __shared__ __align__(8) uint64_t bars[PB_COUNT];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ __align__(16) float s_scale[2][PF_NT];   // dq[m] * w_scale per token column, double-buffered by work item
    __shared__ __align__(16) int s_rs[2][PF_NT];        // code sum per token column

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    pdl_trigger();

    if (tid < PB_COUNT) mbar_init(&bars[tid], pf_bar_count(tid));
    if (tid == PB_COUNT) s_abort = 0;
    if (warp == PF_WARP_MMA) tmem_alloc(&s_tmem_base, 512u);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t tmem_a = tmem_base + PF_NT;
    volatile int* abort_flag = &s_abort;
    const int S = (p.KC + 1) / 2;              // 128-K stages per work item
    const int first = blockIdx.x, step = gridDim.x;

    if (warp == PF_WARP_W) {
        // ------------------------------------------------------------ packed weights (bulk TMA); independent of the
        // preceding kernel, so the stream starts before the grid dependency wait
        if (elect_one()) {
            PfRing w{0, 0, PF_SW};
            bool live = true;
            for (int wk = first; wk < p.n_work && live; wk += step) {
                const int tile = wk % p.n_tiles;
                const uint8_t* src = reinterpret_cast<const uint8_t*>(a.packed) + (int64_t)tile * p.KC * (MMF_TILE_ROWS * 16);
                for (int i = 0; i < S; ++i, w.next()) {
                    const uint32_t bytes = (uint32_t)min(2, p.KC - i * 2) * (MMF_TILE_ROWS * 16);
                    if (!mbar_wait(&bars[PB_W_EMPTY + w.slot], w.ph ^ 1, abort_flag)) { live = false; break; }
                    mbar_expect_tx(&bars[PB_W_FULL + w.slot], bytes);
                    bulk_load_1d(w_ring + w.slot * PF_W_STAGE, src + (int64_t)i * PF_W_STAGE, bytes, &bars[PB_W_FULL + w.slot]);
                }
            }
        }
    } else if (warp == PF_WARP_B) {
        // ------------------------------------------------------------ activation tiles (TMA, 128-byte swizzle)
        pdl_wait();
        if (elect_one()) {
            PfRing bq{0, 0, PF_SB};
            bool live = true;
            for (int wk = first; wk < p.n_work && live; wk += step) {
                const int tile = wk % p.n_tiles, mt = wk / p.n_tiles;
                const int y = (tile / p.group_tiles) * a.M + mt * PF_NT;
                for (int i = 0; i < S; ++i, bq.next()) {
                    if (!mbar_wait(&bars[PB_B_EMPTY + bq.slot], bq.ph ^ 1, abort_flag)) { live = false; break; }
                    mbar_expect_tx(&bars[PB_B_FULL + bq.slot], (uint32_t)PF_B_STAGE);
                    tma_load_2d(b_ring + bq.slot * PF_B_STAGE, &q_map, &bars[PB_B_FULL + bq.slot], i * 128, y);
                }
            }
        }
    } else if (warp == PF_WARP_MMA) {
        // ------------------------------------------------------------ MMA issue: a serial instruction stream, kept short
        if (elect_one()) {
            PfRing bq{0, 0, PF_SB}, aq{0, 0, PF_SA};
            const uint64_t b_desc0 = make_b_desc(smem_u32(b_ring));
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            const uint32_t b_desc_step = (uint32_t)PF_B_STAGE >> 4;
            const int nfull = p.KC / 2;          // whole 128-K stages; a trailing 64-K stage issues two MMAs
            bool live = true;
            int it = 0;
            for (int wk = first; wk < p.n_work && live; wk += step, ++it) {
                // the epilogue must have drained the accumulator of the previous work item
                if (!mbar_wait(&bars[PB_ACC_EMPTY], (uint32_t)((it & 1) ^ 1), abort_flag)) break;
                tc_fence_after();
                uint32_t accum = 0;
                for (int i = 0; i < S; ++i, bq.next(), aq.next()) {
                    if (!mbar_wait(&bars[PB_B_FULL + bq.slot], bq.ph, abort_flag)) { live = false; break; }
                    if (!mbar_wait(&bars[PB_A_FULL + aq.slot], aq.ph, abort_flag)) { live = false; break; }
                    tc_fence_after();
                    uint32_t a_addr = tmem_a + aq.slot * 32;
                    uint32_t b_lo = b_lo0 + (uint32_t)bq.slot * b_desc_step;
                    if (i < nfull) {
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t.reg .b64 d0, d1, d2, d3;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "mov.b64 d0, {%1, %3};\n\t"
                            "add.u32 %1, %1, 2;\n\t"
                            "mov.b64 d1, {%1, %3};\n\t"
                            "add.u32 %1, %1, 2;\n\t"
                            "mov.b64 d2, {%1, %3};\n\t"
                            "add.u32 %1, %1, 2;\n\t"
                            "mov.b64 d3, {%1, %3};\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%2], [%0], d0, %5, p;\n\t"
                            "add.u32 %0, %0, 8;\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%2], [%0], d1, %5, 1;\n\t"
                            "add.u32 %0, %0, 8;\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%2], [%0], d2, %5, 1;\n\t"
                            "add.u32 %0, %0, 8;\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%2], [%0], d3, %5, 1;\n\t}"
                            : "+r"(a_addr), "+r"(b_lo)
                            : "r"(tmem_base), "r"(b_hi), "r"(accum), "r"(p.idesc)
                            : "memory");
                    } else {
                        const uint64_t bd = ((uint64_t)b_hi << 32) | b_lo;
                        mma_i8_ts(tmem_base, a_addr, bd, p.idesc, accum);
                        mma_i8_ts(tmem_base, a_addr + 8, bd + 2, p.idesc, 1u);
                    }
                    accum = 1;
                    tc_commit(&bars[PB_A_EMPTY + aq.slot]);   // frees the A stage when these MMAs retire
                    tc_commit(&bars[PB_B_EMPTY + bq.slot]);
                }
                if (live) tc_commit(&bars[PB_ACC_FULL]);
            }
        }
    } else if (warp < PF_UNPACK_WARPS) {
        // ------------------------------------------------------------ unpack: lane <-> TMEM lane <-> weight row
        const int qd = warp & 3, gp = warp >> 2;
        const int row = qd * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
        PfRing w{0, 0, PF_SW}, aq{0, 0, PF_SA};
        if (gp) { w.next(); aq.next(); }
        int sg = gp;            // next global stage (counted across work items) this group expands
        int tile_base = 0;      // global index of the current work item's first stage
        bool ok = true;
        for (int wk = first; wk < p.n_work && ok; wk += step, tile_base += S) {
            for (; sg < tile_base + S; sg += 2) {
                const int i = sg - tile_base;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars[PB_W_FULL + w.slot], w.ph, abort_flag));   // warp-uniform
                if (!ok) break;
                const int nch = min(2, p.KC - i * 2);
                const uint8_t* wsrc = w_ring + w.slot * PF_W_STAGE + row * 16;
                uint4 wv[2];
                wv[0] = *reinterpret_cast<const uint4*>(wsrc);
                wv[1] = nch > 1 ? *reinterpret_cast<const uint4*>(wsrc + MMF_TILE_ROWS * 16) : wv[0];
                mbar_arrive(&bars[PB_W_EMPTY + w.slot]);          // the packed bytes are in registers now
                ok = __all_sync(0xffffffffu, mbar_wait(&bars[PB_A_EMPTY + aq.slot], aq.ph ^ 1, abort_flag));
                if (!ok) break;   // uniform per warp: the .sync.aligned tcgen05 ops below need the whole warp
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h < nch) {
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
                tc_fence_before();
                mbar_arrive(&bars[PB_A_FULL + aq.slot]);
                w.next(); w.next();
                aq.next(); aq.next();
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: TMEM -> registers -> global memory
        const int ew = warp - PF_UNPACK_WARPS;
        const int lq = ew & 3, hf = ew >> 2;
        const uint32_t lane_addr = (uint32_t)(lq * 32) << 16;
        const int col0 = hf * (PF_NT / 2);
        const int eidx = ew * 32 + lane;              // 0..255: the token column whose constants this thread stages
        pdl_wait();                                   // dq / rowsum come from the preceding kernel
        bool ok = true;
        int it = 0;
        for (int wk = first; wk < p.n_work && ok; wk += step, ++it) {
            const int tile = wk % p.n_tiles, mt = wk / p.n_tiles;
            const int g = tile / p.group_tiles;
            const int m0 = mt * PF_NT;
            float* sc = s_scale[it & 1];
            int* rs = s_rs[it & 1];
            {
                const int m = m0 + eidx;
                const bool in = m < a.M;
                sc[eidx] = in ? __fmul_rn(a.dq[(int64_t)g * a.M + m], a.w_scale[g]) : 0.0f;
                rs[eidx] = in ? a.rowsum[(int64_t)g * a.M + m] : 0;
            }
            asm volatile("bar.sync 1, %0;" ::"n"(PF_EPI_WARPS * 32) : "memory");   // the 8 epilogue warps only
            ok = __all_sync(0xffffffffu, mbar_wait(&bars[PB_ACC_FULL], (uint32_t)(it & 1), abort_flag));
            if (!ok) break;
            tc_fence_after();
            const int n = tile * MMF_TILE_ROWS + lq * 32 + lane;
            const bool n_ok = n < a.N;
            const int mvalid = min(PF_NT / 2, a.M - m0 - col0);    // valid token columns in this warp's half (may be <= 0)
            uint32_t v[2][16];
            tmem_ld16(tmem_base + lane_addr + col0, v[0]);
#pragma unroll
            for (int c = 0; c < PF_NT / 32; ++c) {
                tmem_wait_ld();
                if (c + 1 < PF_NT / 32) {
                    tmem_ld16(tmem_base + lane_addr + col0 + (c + 1) * 16, v[(c + 1) & 1]);
                } else {
                    // the whole accumulator half is in registers: hand it back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[PB_ACC_EMPTY]);
                }
                const int ncols = mvalid - c * 16;
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
    }

    // teardown: everyone meets, TMEM goes back; on the error path give copies in flight time to land first
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
    tc_fence_before();
    __syncthreads();
    if (warp == PF_WARP_MMA) tmem_dealloc(tmem_base, 512u);
}

}  // namespace

// Launch the persistent kernel (large M).  Same argument contract as bitlinear_mma_launch.
int bitlinear_mma_prefill_launch(const BitLinearArgs& a, cudaStream_t st) {
    PfParams p;
    p.KC = a.K / MMF_TILE_K;
    p.n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    p.group_tiles = p.n_tiles / a.groups;
    p.m_tiles = (a.M + PF_NT - 1) / PF_NT;
    const int64_t n_work = (int64_t)p.n_tiles * p.m_tiles;
    MMF_REQUIRE(n_work < (1ll << 31), MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): problem too large");
    p.n_work = (int)n_work;
    // instruction descriptor: D=S32, A=S8 (TMEM), B=S8 (smem, K-major), M=128, N=256
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(PF_NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

    MmfEncodeTiledFn encode = mmf_encode_tiled();
    MMF_REQUIRE(encode != nullptr, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap q_map;
    const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.groups * (cuuint64_t)a.M};
    const cuuint64_t gstride[1] = {(cuuint64_t)a.K};
    const cuuint32_t box[2] = {128u, (cuuint32_t)PF_NT};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult cr = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(a.q), gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MMF_REQUIRE(cr == CUDA_SUCCESS, MMF_ERR_CUDA, "mmf_bitlinear(mma): cuTensorMapEncodeTiled failed (%d)", (int)cr);

    int dev = 0, sms = 0;
    MMF_CUDA(cudaGetDevice(&dev));
    MMF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MMF_CUDA(cudaFuncSetAttribute(bitlinear_mma_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.n_work < sms ? p.n_work : sms));
    cfg.blockDim = dim3(PF_THREADS);
    cfg.dynamicSmemBytes = PF_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MMF_CUDA(cudaLaunchKernelEx(&cfg, bitlinear_mma_prefill_kernel, q_map, a, p));
    MMF_LAUNCH_CHECK("bitlinear_mma_prefill_kernel");
    return MMF_OK;
}
