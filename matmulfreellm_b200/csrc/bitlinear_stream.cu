// BitLinear for a decode step (1 .. 64 token rows): a persistent, latency-lean weight-streaming kernel.
//
// A decode step is a chain of ~100 dependent contractions, each of which moves only a few megabytes of 2-bit weights:
// what counts is the time from "the activation codes exist" to "the outputs are in memory", not throughput.  This
// kernel therefore has no tensor-memory allocation, no cluster, no cross-CTA reduction and no block-wide barrier
// after its set-up:
//
//   * one CTA per SM; the CTA keeps ALL activation codes of its group resident in shared memory ([K/64] chunks of
//     [tokens][64 bytes], fetched once by tiled TMA after the grid-dependency wait) and walks over "slabs" of 16
//     output rows (slab j of CTA b is slab b + j * CTAs of the group), so the codes cross L2 -> SM once per SM;
//   * the 2-bit weights of a slab (K/64 pieces of 256 contiguous bytes) arrive by bulk TMA into a ring of whole
//     slabs.  They do not depend on the preceding kernel: the ring is filled BEFORE the grid-dependency wait
//     (programmatic dependent launch), so after the wait only the codes have to travel;
//   * a warp owns one (slab, 8-token tile) pair and contracts it over the whole of K with mma.sync m16n8k32
//     (s8 x s8 -> s32): the A fragment (16 weight rows x 32 columns) is two 32-bit words of packed weights per
//     thread, expanded with shift + mask in registers ((word >> 2i) & 0x03030303 is four consecutive columns as
//     bytes), the B fragment is one 16-byte shared-memory load of codes per 64 columns.  The K order inside an MMA
//     is permuted identically for both operands, so no data is rearranged.  Warps of different slabs or token tiles
//     never exchange data; each writes its own outputs;
//   * measured on B200: mma.sync.m16n8k32.s8 sustains 4096 op/clk/SM (1.14 POP/s per GPU), so a 32-token step of
//     a 1.3 B-parameter model needs about 75 us of tensor-pipe time — the same order as the 50 us its weight stream
//     needs from HBM; tcgen05 would not make a 32-column tile faster, and costs a TMEM round trip per tile.
//
// Weights are stored biased (+1): the epilogue subtracts the row's code sum, then dequantises (acc * (dq * mean|w|)).
// Every wait is bounded; a wait that gives up sets the status word of the workspace (if one was passed).
#include <cuda.h>

#include "bitlinear.cuh"
#include "tensor_map.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int SK_COMPUTE_WARPS = 8;
constexpr int SK_WARP_W = 8;       // packed-weight producer
constexpr int SK_WARP_C = 9;       // activation-code producer
constexpr int SK_THREADS = 10 * 32;
constexpr int SK_MAX_CODE_GROUPS = 32;   // barriers for groups of 4 chunks (256 columns): K <= 8192
constexpr int SK_MAX_SLOTS = 8;          // weight ring: whole slabs
constexpr int SK_SLAB_ROWS = 16;
constexpr int SK_PIECE = SK_SLAB_ROWS * 16;   // bytes of one slab x one 64-column chunk

struct StreamParams {
    int KC;              // K / 64
    int MT;              // 8-token tiles (M padded to 8 * MT)
    int SL;              // slabs a CTA works on at a time = compute warps / MT
    int slabs_per_group; // ceil((N / groups) / 16)
    int tiles_per_group; // 128-row weight tiles per group
    int ctas_per_group;
    int slots;           // weight ring depth (slabs)
    int code_groups;     // ceil(KC / 4)
    int m0, mb;          // token rows [m0, m0 + mb) of every group are this launch's share (mb <= 8 * MT)
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// two consecutive outputs (n, n+1) of token m
__device__ __forceinline__ void store_pair(const BitLinearArgs& a, int m, int n, int v0, int v1, float scale, bool pair_ok) {
    if (n >= a.N) return;
    const bool both = n + 1 < a.N;
    if (a.acc_out) {
        a.acc_out[(int64_t)m * a.N + n] = v0;
        if (both) a.acc_out[(int64_t)m * a.N + n + 1] = v1;
    }
    const float f0 = __fmul_rn((float)v0, scale), f1 = __fmul_rn((float)v1, scale);
    const int64_t off = (int64_t)m * a.ld_out + n;
    if (both && pair_ok) {
        if (a.out_dtype == MMF_F32) {
            *reinterpret_cast<float2*>(reinterpret_cast<float*>(a.out) + off) = make_float2(f0, f1);
        } else if (a.out_dtype == MMF_BF16) {
            *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(a.out) + off) = __floats2bfloat162_rn(f0, f1);
        } else {
            *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(a.out) + off) = __floats2half2_rn(f0, f1);
        }
    } else {
        store_out(a.out, a.out_dtype, off, f0);
        if (both) store_out(a.out, a.out_dtype, off + 1, f1);
    }
}

__global__ void __launch_bounds__(SK_THREADS, 1)
bitlinear_stream_kernel(const __grid_constant__ CUtensorMap q_map, BitLinearArgs a, StreamParams p, int pair_ok) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int m_pad = p.MT * 8;
    const int chunk_bytes = m_pad * 64;                    // codes of one 64-column chunk: [token][64]
    uint8_t* codes = base;                                 // [KC][m_pad][64]
    const int slab_bytes = p.KC * SK_PIECE;                // [KC][16 rows][16 bytes]
    uint8_t* wring = base + (size_t)p.KC * chunk_bytes;    // [slots][slab_bytes]

    __shared__ __align__(8) uint64_t bar_code[SK_MAX_CODE_GROUPS];
    __shared__ __align__(8) uint64_t bar_wfull[SK_MAX_SLOTS];
    __shared__ __align__(8) uint64_t bar_wempty[SK_MAX_SLOTS];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    pdl_trigger();   // the next kernel may start its own set-up right away
    const int g = blockIdx.x % a.groups, cb = blockIdx.x / a.groups;
    // this CTA's slabs of group g: cb, cb + ctas_per_group, ...
    const int nj = cb < p.slabs_per_group ? (p.slabs_per_group - 1 - cb) / p.ctas_per_group + 1 : 0;

    if (tid < SK_MAX_CODE_GROUPS) mbar_init(&bar_code[tid], 1);
    else if (tid < SK_MAX_CODE_GROUPS + SK_MAX_SLOTS) mbar_init(&bar_wfull[tid - SK_MAX_CODE_GROUPS], 1);
    else if (tid < SK_MAX_CODE_GROUPS + 2 * SK_MAX_SLOTS) mbar_init(&bar_wempty[tid - SK_MAX_CODE_GROUPS - SK_MAX_SLOTS], (uint32_t)p.MT);
    if (tid == SK_THREADS - 1) s_abort = 0;
    if (tid == SK_WARP_C * 32) prefetch_tensormap(&q_map);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    volatile int* abort_flag = &s_abort;

    if (warp == SK_WARP_W) {
        // ------------------------------------------------------------ packed weights: whole slabs, before the dependency wait
        for (int j = 0; j < nj; ++j) {
            const int slot = j % p.slots, use = j / p.slots;
            bool ok = true;
            if (use > 0 && lane == 0) ok = mbar_wait_relaxed(&bar_wempty[slot], (uint32_t)(use - 1) & 1u, abort_flag);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(&bar_wfull[slot], (uint32_t)slab_bytes);
            __syncwarp();
            const int slab = cb + j * p.ctas_per_group;                       // slab of group g
            const int tile = g * p.tiles_per_group + (slab >> 3), r0 = (slab & 7) * SK_SLAB_ROWS;
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.packed) + ((int64_t)tile * p.KC * MMF_TILE_ROWS + r0) * 16;
            uint8_t* dst = wring + (size_t)slot * slab_bytes;
            for (int c = lane; c < p.KC; c += 32)
                bulk_load_1d(dst + c * SK_PIECE, src + (int64_t)c * (MMF_TILE_ROWS * 16), SK_PIECE, &bar_wfull[slot]);
        }
    } else if (warp == SK_WARP_C) {
        // ------------------------------------------------------------ activation codes: the preceding kernel's output
        pdl_wait();
        if (nj > 0) {
            if (lane < p.code_groups) {
                const int nch = min(4, p.KC - lane * 4);
                mbar_expect_tx(&bar_code[lane], (uint32_t)(nch * chunk_bytes));
            }
            __syncwarp();
            const int y = g * a.M + p.m0;
            for (int c = lane; c < p.KC; c += 32)
                tma_load_2d(codes + (size_t)c * chunk_bytes, &q_map, &bar_code[c >> 2], c * 64, y);
        }
    } else {
        // ------------------------------------------------------------ compute: warp = (slab lane, token tile)
        const int nt = warp % p.MT, sl = warp / p.MT;
        if (sl < p.SL) {
            const int gq = lane >> 2, t = lane & 3;          // fragment coordinates: row / token gq, K quad t
            // after the exchange below a thread finishes ONE token: columns (2t, 2t+1) of the tile -> token 2t + (gq & 1)
            const int ml = nt * 8 + 2 * t + (gq & 1), m = p.m0 + ml;
            const bool live = ml < p.mb;
            pdl_wait();                                      // dq / rowsum are the preceding kernel's output
            float scale = 0.0f;
            int rsum = 0;
            if (live) {
                scale = __fmul_rn(a.dq[(int64_t)g * a.M + m], a.w_scale[g]);
                rsum = a.rowsum[(int64_t)g * a.M + m];
            }
            const uint8_t* bsrc = codes + (size_t)(nt * 8 + gq) * 64 + 16 * t;
            bool ok = true;
            for (int j = sl; j < nj && ok; j += p.SL) {
                const int slot = j % p.slots, use = j / p.slots;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar_wfull[slot], (uint32_t)use & 1u, abort_flag));
                if (!ok) break;
                const uint32_t* wsm = reinterpret_cast<const uint32_t*>(wring + (size_t)slot * slab_bytes) + gq * 4 + t;
                int accA[4] = {0, 0, 0, 0}, accB[4] = {0, 0, 0, 0};
                for (int cg = 0; cg < p.code_groups && ok; ++cg) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bar_code[cg], 0u, abort_flag));   // completes once; later slabs pass at once
                    if (!ok) break;
                    const int c0 = cg * 4, nch = min(4, p.KC - c0);
#pragma unroll
                    for (int ci = 0; ci < 4; ++ci) {
                        if (ci < nch) {
                            const int c = c0 + ci;
                            const uint32_t lo = wsm[c * (SK_PIECE / 4)], hi = wsm[c * (SK_PIECE / 4) + 32];   // rows gq, gq + 8
                            const uint4 b = *reinterpret_cast<const uint4*>(bsrc + (size_t)c * chunk_bytes);
                            mma_s8(accA, lo & 0x03030303u, hi & 0x03030303u, (lo >> 2) & 0x03030303u, (hi >> 2) & 0x03030303u, b.x, b.y);
                            mma_s8(accB, (lo >> 4) & 0x03030303u, (hi >> 4) & 0x03030303u, (lo >> 6) & 0x03030303u,
                                   (hi >> 6) & 0x03030303u, b.z, b.w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_wempty[slot]);   // this warp has read the slab's weights
                if (!ok) break;
                // C fragment: c0/c1 = (row gq, tokens 2t, 2t+1), c2/c3 = (row gq + 8, same tokens).  Lanes gq and gq^1
                // swap so that each thread holds two consecutive rows of one token: one 4-byte (or 8-byte) store each.
                const int v0 = accA[0] + accB[0], v1 = accA[1] + accB[1], v2 = accA[2] + accB[2], v3 = accA[3] + accB[3];
                const bool odd = gq & 1;
                const int sx = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 4);
                const int sy = __shfl_xor_sync(0xffffffffu, odd ? v2 : v3, 4);
                if (live) {
                    const int slab = cb + j * p.ctas_per_group;
                    // output row index inside the whole [M, N] output: group g's rows start at g * (N / groups)
                    const int n = g * (a.N / a.groups) + slab * SK_SLAB_ROWS + (gq & ~1);
                    const int lo0 = (odd ? sx : v0) - rsum, lo1 = (odd ? v1 : sx) - rsum;
                    const int hi0 = (odd ? sy : v2) - rsum, hi1 = (odd ? v3 : sy) - rsum;
                    const int n_end = g * (a.N / a.groups) + min(a.N / a.groups, (slab + 1) * SK_SLAB_ROWS);   // rows of this group only
                    if (n < n_end) store_pair(a, m, n, lo0, lo1, scale, pair_ok && n + 1 < n_end);
                    if (n + 8 < n_end) store_pair(a, m, n + 8, hi0, hi1, scale, pair_ok && n + 9 < n_end);
                }
            }
        }
    }

    // teardown: on the error path give copies in flight time to land before the CTA (and its shared memory) goes away
    __syncthreads();
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
}

int g_num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n = v;
        else n = 148;
    }
    return n;
}

}  // namespace

// Token rows one launch can take: the codes of all of them ([K/64][rows][64] bytes) stay in shared memory beside at
// least one slab of weights.  More rows (up to MMF_STREAM_MAX_M) run as several launches over blocks of rows.
static int stream_rows_per_launch(int K) {
    const int KC = K / MMF_TILE_K;
    const size_t slab = (size_t)KC * SK_PIECE;
    const size_t room = 220 * 1024 - 1024 - slab;
    int rows = (int)(room / ((size_t)KC * 64)) & ~7;
    return rows > 64 ? 64 : rows;
}

// true if the streaming kernel can take this problem
bool bitlinear_stream_fits(const BitLinearArgs& a) {
    return a.M <= MMF_STREAM_MAX_M && a.K <= SK_MAX_CODE_GROUPS * 256 && stream_rows_per_launch(a.K) >= 8;
}

int bitlinear_stream_launch(const BitLinearArgs& a, cudaStream_t st) {
    MMF_REQUIRE(bitlinear_stream_fits(a), MMF_ERR_BAD_SHAPE, "mmf_bitlinear(stream): M=%d K=%d does not fit the decode kernel", a.M, a.K);
    const int cap = stream_rows_per_launch(a.K);
    const int blocks = (a.M + cap - 1) / cap;
    const int rows_per_block = (((a.M + blocks - 1) / blocks) + 7) & ~7;   // balanced, whole 8-token tiles

    MmfEncodeTiledFn encode = mmf_encode_tiled();
    MMF_REQUIRE(encode != nullptr, MMF_ERR_CUDA, "mmf_bitlinear(stream): cuTensorMapEncodeTiled is not available from the driver");
    static bool attr_set = false;
    if (!attr_set) {
        MMF_CUDA(cudaFuncSetAttribute(bitlinear_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)));
        attr_set = true;
    }
    // paired stores need an even leading dimension and an aligned base
    const int es = mmf_dtype_size(a.out_dtype);
    const int pair_ok = (a.ld_out % 2 == 0) && mmf_aligned(a.out, (size_t)2 * es) && (a.N / a.groups) % 2 == 0 ? 1 : 0;
    const int sms = g_num_sms();
    const int n_group = a.N / a.groups;

    for (int m0 = 0; m0 < a.M; m0 += rows_per_block) {
        StreamParams p;
        p.KC = a.K / MMF_TILE_K;
        p.m0 = m0;
        p.mb = a.M - m0 < rows_per_block ? a.M - m0 : rows_per_block;
        p.MT = (p.mb + 7) / 8;
        p.SL = SK_COMPUTE_WARPS / p.MT;
        p.slabs_per_group = (n_group + SK_SLAB_ROWS - 1) / SK_SLAB_ROWS;
        p.tiles_per_group = (n_group + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
        p.ctas_per_group = sms / a.groups < 1 ? 1 : sms / a.groups;
        if (p.ctas_per_group > p.slabs_per_group) p.ctas_per_group = p.slabs_per_group;
        p.code_groups = (p.KC + 3) / 4;
        const size_t codes = (size_t)p.KC * p.MT * 8 * 64, slab = (size_t)p.KC * SK_PIECE;
        const int max_j = (p.slabs_per_group + p.ctas_per_group - 1) / p.ctas_per_group;
        // Kernels of a decode step start while their predecessors still run (programmatic dependent launch) and use that
        // time to fetch their weights, which only works if both fit on an SM side by side: stay under ~108 KB when one
        // slab beside the codes allows it, otherwise take what a single CTA may have.
        const size_t budget = codes + slab + 1024 <= 108 * 1024 ? 108 * 1024 : 220 * 1024;
        int slots = (int)((budget - 1024 - codes) / slab);
        if (slots > max_j) slots = max_j;
        if (slots > SK_MAX_SLOTS) slots = SK_MAX_SLOTS;
        p.slots = slots;
        const size_t smem = 128 + codes + (size_t)slots * slab;

        CUtensorMap q_map;
        const cuuint64_t gdim[2] = {(cuuint64_t)a.K, (cuuint64_t)a.groups * (cuuint64_t)a.M};
        const cuuint64_t gstride[1] = {(cuuint64_t)a.K};
        const cuuint32_t box[2] = {64u, (cuuint32_t)(p.MT * 8)};
        const cuuint32_t estr[2] = {1u, 1u};
        const CUresult cr = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(a.q), gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MMF_REQUIRE(cr == CUDA_SUCCESS, MMF_ERR_CUDA, "mmf_bitlinear(stream): cuTensorMapEncodeTiled failed (%d)", (int)cr);
        const dim3 grid((unsigned)(p.ctas_per_group * a.groups));
        MMF_CUDA(mmf_launch_pdl(bitlinear_stream_kernel, grid, dim3(SK_THREADS), smem, st, q_map, a, p, pair_ok));
        MMF_LAUNCH_CHECK("bitlinear_stream_kernel");
    }
    return MMF_OK;
}
