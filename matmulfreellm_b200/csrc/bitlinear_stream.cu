// BitLinear for a decode step (1 .. 64 token rows) as a persistent weight-streaming kernel on mma.sync — an EXPERIMENT,
// compiled only into the experiments build (-DMMF_EXPERIMENTS); the product library does not contain it.
//
// Question it answers: a decode step is a chain of ~100 dependent contractions of a few megabytes each; would a kernel
// with no tensor-memory allocation, no cluster and no cross-CTA reduction beat the tcgen05 kernel (bitlinear_mma.cu) and
// the dp4a GEMV (bitlinear_gemv.cu) on latency?  Design:
//
//   * one CTA per SM; the CTA keeps ALL activation codes of its group resident in shared memory ([K/64] chunks of
//     [tokens][64 bytes], copied once with cp.async after the grid-dependency wait) and walks over "slabs" of 16
//     output rows (slab j of CTA b is slab b + j * CTAs of the group), so the codes cross L2 -> SM once per SM;
//   * the 2-bit weights are read from a SLAB-MAJOR copy of the packed weight (mmf_repack_slabs): a slab's K/4 * 16
//     bytes are contiguous, so one bulk-TMA copy fetches a whole slab into a ring of slabs, filled BEFORE the
//     grid-dependency wait (programmatic dependent launch).  (256-byte pieces of the tile-major layout, one bulk copy
//     each, were measured first: the copy engine then bounds the launch at ~8 us whatever the token count.)
//   * four warps share a slab, each contracting every fourth 64-column chunk against ALL token tiles with mma.sync
//     m16n8k32 (s8 x s8 -> s32): the A fragment (16 weight rows x 32 columns) is two 32-bit words of packed weights
//     per thread, expanded with shift + mask in registers, the B fragment one 16-byte shared-memory load of codes per
//     token tile and chunk; the K order inside an MMA is permuted identically for both operands.  The four partial
//     sums meet in shared memory (one named barrier of 128 threads); two slabs are in flight per CTA.
//
// Answer (measured on B200, HGRNBit-1.3B decode steps replayed from a CUDA graph): no.  A bare mma.sync.m16n8k32.s8 loop
// sustains 4096 op/clk/SM, but with the 2-bit expansion and the shared-memory operand loads a warp issues one MMA per
// ~23 cycles (188 - 215 cycles per 64-column chunk of 8 MMAs: shared-memory bandwidth for the codes and the issue slots
// of the expansion bound it together), i.e. ~700 MAC/clk/SM at 32 tokens where the tcgen05 kernel reaches ~1950.  Whole
// steps: batch 1: 0.69 ms (GEMV 0.62), batch 4: 0.79 (GEMV 0.84, tcgen05 ~0.75), batch 8: 0.82 (tcgen05 0.75), batch 32:
// 1.06 (tcgen05 0.84).  Per launch inside the chain (timeline of CTA 0): 1.1 - 3.5 us from the predecessor's end to the
// release of the grid dependency, 0.3 - 1.1 us for the codes, 0.4 - 2.4 us per slab.
//
// Weights are stored biased (+1): the epilogue subtracts the row's code sum, then dequantises (acc * (dq * mean|w|)).
// Every wait is bounded; a wait that gives up sets the status word (if one was passed).
#ifdef MMF_EXPERIMENTS
#include "../../include/mmfree_b200_experiments.h"
#include "bitlinear.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int SK_COMPUTE_WARPS = 8;
constexpr int SK_KP = 4;                 // warps sharing one slab (K split)
constexpr int SK_WARP_W = SK_COMPUTE_WARPS;           // packed-weight producer warp
constexpr int SK_THREADS = (SK_COMPUTE_WARPS + 1) * 32;
constexpr int SK_MAX_SLOTS = 8;          // weight ring: whole slabs
constexpr int SK_SLAB_ROWS = 16;
constexpr int SK_PIECE = SK_SLAB_ROWS * 16;   // bytes of one slab x one 64-column chunk

struct StreamParams {
    int KC;              // K / 64
    int SL;              // slabs a CTA works on at a time (1 or 2)
    int depth;           // ring slots per slab lane
    int slabs_per_group; // ceil((N / groups) / 16)
    int tiles_per_group; // 128-row weight tiles per group
    int ctas_per_group;
    int m0, mb;          // token rows [m0, m0 + mb) of every group are this launch's share (mb <= 8 * MT)
};

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    // not volatile: a pure function of its operands, so the compiler may interleave it with the loads of later chunks
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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

// Timeline trace of CTA 0 for kernel experiments (experiments build only; folds away in the product build): when word 1
// of the status buffer holds MMF_TRACE_MAGIC, every launch takes a record of 8 global-timer stamps (nanoseconds) at
// status + 16 + 16 * (launch index from an atomic counter in word 2).
#ifdef MMF_EXPERIMENTS
__device__ __forceinline__ long long sk_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define SK_TRACE(slot) do { if (trace) trace[slot] = sk_now(); } while (0)
#else
#define SK_TRACE(slot) do { } while (0)
#endif

template <int MT>   // token tiles of 8 (tokens padded to 8 * MT)
__global__ void __launch_bounds__(SK_THREADS, 1)
bitlinear_stream_kernel(BitLinearArgs a, const uint8_t* __restrict__ slabs, StreamParams p, int pair_ok) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    constexpr int M_PAD = MT * 8;
    constexpr int CHUNK_BYTES = M_PAD * 64;                // codes of one 64-column chunk: [token][64]
    constexpr int OWN = (MT + SK_KP - 1) / SK_KP;          // token tiles a warp finishes (tiles kp, kp + 4)
    uint8_t* codes = base;                                 // [KC][M_PAD][64]
    const int slab_bytes = p.KC * SK_PIECE;                // [KC][16 rows][16 bytes]
    uint8_t* wring = base + (size_t)p.KC * CHUNK_BYTES;    // [SL * depth][slab_bytes]
    int* red = reinterpret_cast<int*>(wring + (size_t)p.SL * p.depth * slab_bytes);   // [SL][KP][MT][4][32]

    __shared__ __align__(8) uint64_t bar_wfull[SK_MAX_SLOTS];
    __shared__ __align__(8) uint64_t bar_wempty[SK_MAX_SLOTS];
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef MMF_EXPERIMENTS
    __shared__ long long* s_trace;
    if (tid == 0) {
        s_trace = nullptr;
        if (blockIdx.x == 0 && a.ws && a.ws[1] == MMF_TRACE_MAGIC) {
            const int idx = atomicAdd(a.ws + 2, 1);
            a.ws[3] = idx;
            if (idx < 4000) s_trace = reinterpret_cast<long long*>(a.ws + 16) + 8 * idx;
        }
        if (s_trace) s_trace[0] = sk_now();
    }
#endif
    pdl_trigger();   // the next kernel may start its own set-up right away
    const int g = blockIdx.x % a.groups, cb = blockIdx.x / a.groups;
    // this CTA's slabs of group g: cb, cb + ctas_per_group, ...
    const int nj = cb < p.slabs_per_group ? (p.slabs_per_group - 1 - cb) / p.ctas_per_group + 1 : 0;

    if (tid < SK_MAX_SLOTS) mbar_init(&bar_wfull[tid], 1);
    else if (tid < 2 * SK_MAX_SLOTS) mbar_init(&bar_wempty[tid - SK_MAX_SLOTS], SK_KP);
    if (tid == SK_THREADS - 1) s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    volatile int* abort_flag = &s_abort;
#ifdef MMF_EXPERIMENTS
    long long* const trace = (tid == 0 || tid == SK_WARP_W * 32) ? s_trace : nullptr;
#endif
    if (tid == 0) SK_TRACE(1);

    if (warp == SK_WARP_W) {
        // ------------------------------------------------------------ packed weights: one bulk copy per slab, started
        // before the grid-dependency wait (weights are constants)
        if (lane == 0) {
            for (int j = 0; j < nj; ++j) {
                const int sl = j % p.SL, jj = j / p.SL;
                const int slot = sl * p.depth + jj % p.depth, use = jj / p.depth;
                if (use > 0 && !mbar_wait_relaxed(&bar_wempty[slot], (uint32_t)(use - 1) & 1u, abort_flag)) break;
                const int64_t slab = (int64_t)g * p.tiles_per_group * (MMF_TILE_ROWS / SK_SLAB_ROWS) + cb + (int64_t)j * p.ctas_per_group;
                mbar_expect_tx(&bar_wfull[slot], (uint32_t)slab_bytes);
                bulk_load_1d(wring + (size_t)slot * slab_bytes, slabs + slab * slab_bytes, (uint32_t)slab_bytes, &bar_wfull[slot]);
            }
        }
    } else {
        // ------------------------------------------------------------ compute warps
        const int kp = warp & (SK_KP - 1), sl = warp / SK_KP;
        const int gq = lane >> 2, t = lane & 3;          // fragment coordinates: row / token gq, K quad t
        pdl_wait();                                      // codes, dq and rowsum are the preceding kernel's output
        SK_TRACE(2);
        if (nj > 0) {
            // all codes of this launch's token rows: global [row][K] -> shared [chunk][row][64]
            const int8_t* qsrc = a.q + ((int64_t)g * a.M + p.m0) * a.K;
            const int units = a.K >> 4;                  // 16-byte units per row
            for (int row = warp; row < p.mb; row += SK_COMPUTE_WARPS) {
                const int8_t* src = qsrc + (int64_t)row * a.K;
                uint8_t* dst = codes + row * 64;
                for (int u = lane; u < units; u += 32) cp_async16(dst + (u >> 2) * CHUNK_BYTES + (u & 3) * 16, src + u * 16);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        // per-token constants of the token tiles this warp finishes: after the lane exchange of the epilogue a thread
        // holds ONE token of a tile: columns (2t, 2t+1) -> token 2t + (gq & 1)
        float scale[OWN];
        int rsum[OWN];
        bool live[OWN];
#pragma unroll
        for (int o = 0; o < OWN; ++o) {
            const int ml = (kp + o * SK_KP) * 8 + 2 * t + (gq & 1);
            live[o] = kp + o * SK_KP < MT && ml < p.mb;
            scale[o] = 0.0f;
            rsum[o] = 0;
            if (live[o]) {
                scale[o] = __fmul_rn(a.dq[(int64_t)g * a.M + p.m0 + ml], a.w_scale[g]);
                rsum[o] = a.rowsum[(int64_t)g * a.M + p.m0 + ml];
            }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        named_barrier(1, SK_COMPUTE_WARPS * 32);         // every compute warp's share of the codes has landed
        SK_TRACE(3);

        if (sl < p.SL) {
            const uint8_t* bsrc = codes + gq * 64 + 16 * t;
            const int n_group = a.N / a.groups, n_base = g * n_group;
            bool ok = true;
            int jj = 0;
            for (int j = sl; j < nj && ok; j += p.SL, ++jj) {
                const int slot = sl * p.depth + jj % p.depth, use = jj / p.depth;
                ok = __all_sync(0xffffffffu, mbar_wait(&bar_wfull[slot], (uint32_t)use & 1u, abort_flag));
                if (!ok) break;
                if (jj == 0) SK_TRACE(4);
                const uint32_t* wsm = reinterpret_cast<const uint32_t*>(wring + (size_t)slot * slab_bytes) + gq * 4 + t;
                // A dependent mma.sync waits for its predecessor (measured: a chain of 8 per accumulator made a slab take
                // ~1 us where the tensor pipe needs 0.27), so every warp keeps 16 independent accumulators: the two K steps
                // of a chunk, the MT token tiles, and CS = 8 / MT consecutive chunks of the warp go to different ones.
                constexpr int CS = MT >= 8 ? 1 : 8 / MT;
                int acc[CS][2][MT][4];
#pragma unroll
                for (int s2 = 0; s2 < CS; ++s2)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int nt = 0; nt < MT; ++nt) acc[s2][h][nt][0] = acc[s2][h][nt][1] = acc[s2][h][nt][2] = acc[s2][h][nt][3] = 0;
                auto chunk = [&](int c, int (&accs)[2][MT][4]) {
                    const uint32_t lo = wsm[c * (SK_PIECE / 4)], hi = wsm[c * (SK_PIECE / 4) + 32];   // rows gq, gq + 8
                    const uint32_t a0 = lo & 0x03030303u, a1 = hi & 0x03030303u, a2 = (lo >> 2) & 0x03030303u,
                                   a3 = (hi >> 2) & 0x03030303u, a4 = (lo >> 4) & 0x03030303u, a5 = (hi >> 4) & 0x03030303u,
                                   a6 = (lo >> 6) & 0x03030303u, a7 = (hi >> 6) & 0x03030303u;
                    const uint8_t* bc = bsrc + (size_t)c * CHUNK_BYTES;
#pragma unroll
                    for (int nt = 0; nt < MT; ++nt) {
                        const uint4 b = *reinterpret_cast<const uint4*>(bc + nt * 512);
                        mma_s8(accs[0][nt], a0, a1, a2, a3, b.x, b.y);
                        mma_s8(accs[1][nt], a4, a5, a6, a7, b.z, b.w);
                    }
                };
                for (int c = kp; c < p.KC; c += CS * SK_KP) {
#pragma unroll
                    for (int s2 = 0; s2 < CS; ++s2)
                        if (c + s2 * SK_KP < p.KC) chunk(c + s2 * SK_KP, acc[s2]);
                }
                __syncwarp();
                if (jj == 0) SK_TRACE(5);
                if (lane == 0) mbar_arrive(&bar_wempty[slot]);   // this warp has read the slab's weights
                // the four K parts meet in shared memory: [kp][tile][register][lane]
                int* const myred = red + (size_t)sl * (SK_KP * MT * 128);
#pragma unroll
                for (int nt = 0; nt < MT; ++nt)
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        int v = 0;
#pragma unroll
                        for (int s2 = 0; s2 < CS; ++s2) v += acc[s2][0][nt][r] + acc[s2][1][nt][r];
                        myred[((kp * MT + nt) * 4 + r) * 32 + lane] = v;
                    }
                named_barrier(2 + sl, SK_KP * 32);
                const int slab = cb + j * p.ctas_per_group;
#pragma unroll
                for (int o = 0; o < OWN; ++o) {
                    const int nt = kp + o * SK_KP;
                    if (nt < MT) {                                   // warp-uniform
                        int v[4];
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
                            int s = 0;
#pragma unroll
                            for (int k2 = 0; k2 < SK_KP; ++k2) s += myred[((k2 * MT + nt) * 4 + r) * 32 + lane];
                            v[r] = s;
                        }
                        // C fragment: v0/v1 = (row gq, tokens 2t, 2t+1), v2/v3 = (row gq + 8, same tokens).  Lanes gq and
                        // gq^1 swap so that each thread holds two consecutive rows of one token: one 4- or 8-byte store each.
                        const bool odd = gq & 1;
                        const int sx = __shfl_xor_sync(0xffffffffu, odd ? v[0] : v[1], 4);
                        const int sy = __shfl_xor_sync(0xffffffffu, odd ? v[2] : v[3], 4);
                        if (live[o]) {
                            const int m = p.m0 + nt * 8 + 2 * t + (gq & 1);
                            const int n = n_base + slab * SK_SLAB_ROWS + (gq & ~1);
                            const int n_end = n_base + min(n_group, (slab + 1) * SK_SLAB_ROWS);   // rows of this group only
                            const int lo0 = (odd ? sx : v[0]) - rsum[o], lo1 = (odd ? v[1] : sx) - rsum[o];
                            const int hi0 = (odd ? sy : v[2]) - rsum[o], hi1 = (odd ? v[3] : sy) - rsum[o];
                            if (n < n_end) store_pair(a, m, n, lo0, lo1, scale[o], pair_ok && n + 1 < n_end);
                            if (n + 8 < n_end) store_pair(a, m, n + 8, hi0, hi1, scale[o], pair_ok && n + 9 < n_end);
                        }
                    }
                }
                if (j + p.SL < nj) named_barrier(2 + sl, SK_KP * 32);   // the partial sums are free for the next slab
            }
        }
    }

    // teardown: on the error path give copies in flight time to land before the CTA (and its shared memory) goes away
    if (tid == 0) SK_TRACE(6);
    __syncthreads();
    if (tid == 0) SK_TRACE(7);
#ifdef MMF_EXPERIMENTS
    // end time of EVERY CTA of the first 64 traced launches: [launch][256] at byte offset 512 KB of the status buffer
    if (tid == 0 && a.ws && a.ws[1] == MMF_TRACE_MAGIC && blockIdx.x < 256) {
        const int idx = a.ws[3];     // launch index published by CTA 0 (may lag by one launch for CTAs that end before CTA 0 starts)
        if (idx >= 0 && idx < 64) reinterpret_cast<long long*>(a.ws + 131072)[idx * 256 + blockIdx.x] = sk_now();
    }
#endif
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
}

// re-order the tile-major packed weight ([tile][chunk][128 rows][16 B]) into slab-major ([tile][slab of 16 rows][chunk][16 rows][16 B])
__global__ void repack_slabs_kernel(const uint4* __restrict__ packed, uint4* __restrict__ out, int64_t n_units, int KC) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_units; i += (int64_t)gridDim.x * blockDim.x) {
        // destination index i = ((tile * 8 + s) * KC + c) * 16 + r
        const int r = (int)(i & 15);
        const int64_t q1 = i >> 4;
        const int c = (int)(q1 % KC);
        const int64_t q2 = q1 / KC;
        const int s = (int)(q2 & 7);
        const int64_t tile = q2 >> 3;
        out[i] = packed[(tile * KC + c) * MMF_TILE_ROWS + s * SK_SLAB_ROWS + r];
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

constexpr size_t SK_SMEM_MAX = 220 * 1024;

// shared memory of one launch: codes + ring + partial sums (+ alignment slack)
size_t stream_smem(int KC, int MT, int SL, int depth) {
    return 128 + (size_t)KC * MT * 8 * 64 + (size_t)SL * depth * KC * SK_PIECE + (size_t)SL * SK_KP * MT * 128 * sizeof(int);
}

// Token rows one launch can take: the codes of all of them stay in shared memory beside at least one slab of weights.
// More rows (up to MMF_STREAM_MAX_M) run as several launches over blocks of rows.
int stream_rows_per_launch(int K) {
    const int KC = K / MMF_TILE_K;
    for (int MT = 8; MT >= 1; MT >>= 1)
        if (stream_smem(KC, MT, 1, 1) <= SK_SMEM_MAX) return MT * 8;
    return 0;
}

}  // namespace

// true if the decode kernel can take this problem
static bool bitlinear_stream_fits(const BitLinearArgs& a) {
    return a.M <= MMF_STREAM_MAX_M && stream_rows_per_launch(a.K) >= 8;
}

extern "C" int mmf_bitlinear_decode_fits(int64_t M, int64_t K) {
    if (M < 0 || K <= 0 || K % MMF_TILE_K || K > 65536) return 0;
    return M <= MMF_STREAM_MAX_M && stream_rows_per_launch((int)K) >= 8 ? 1 : 0;
}

extern "C" int mmf_repack_slabs(const void* packed, int64_t N, int64_t K, void* slabs, void* stream) {
    MMF_REQUIRE(packed && slabs, MMF_ERR_BAD_ARG, "mmf_repack_slabs: null pointer");
    MMF_REQUIRE(N > 0 && K > 0 && K % MMF_TILE_K == 0, MMF_ERR_BAD_SHAPE, "mmf_repack_slabs: need K %% 64 == 0 (N=%lld K=%lld)",
                (long long)N, (long long)K);
    MMF_REQUIRE(mmf_aligned(packed, 16) && mmf_aligned(slabs, 16), MMF_ERR_ALIGN, "mmf_repack_slabs: buffers must be 16-byte aligned");
    const int64_t tiles = (N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const int KC = (int)(K / MMF_TILE_K);
    const int64_t n_units = tiles * KC * MMF_TILE_ROWS;
    const int threads = 256;
    const int64_t want = (n_units + threads - 1) / threads;
    const unsigned blocks = (unsigned)(want < 148 * 16 ? want : 148 * 16);
    repack_slabs_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint4*)packed, (uint4*)slabs, n_units, KC);
    MMF_LAUNCH_CHECK("repack_slabs_kernel");
    return MMF_OK;
}

static int bitlinear_stream_launch(const BitLinearArgs& a, const void* slabs, cudaStream_t st) {
    MMF_REQUIRE(bitlinear_stream_fits(a), MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear_decode: M=%d K=%d is outside the decode kernel's range (M <= %d, codes of 8 rows + one slab in shared memory)",
                a.M, a.K, MMF_STREAM_MAX_M);
    const int cap = stream_rows_per_launch(a.K);
    const int blocks = (a.M + cap - 1) / cap;
    const int rows_per_block = (((a.M + blocks - 1) / blocks) + 7) & ~7;   // balanced, whole 8-token tiles
    const int KC = a.K / MMF_TILE_K;

    static bool attr_set = false;
    if (!attr_set) {
        MMF_CUDA(cudaFuncSetAttribute(bitlinear_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)));
        MMF_CUDA(cudaFuncSetAttribute(bitlinear_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)));
        MMF_CUDA(cudaFuncSetAttribute(bitlinear_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)));
        MMF_CUDA(cudaFuncSetAttribute(bitlinear_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(222 * 1024)));
        attr_set = true;
    }
    // paired stores need an even leading dimension and an aligned base
    const int es = mmf_dtype_size(a.out_dtype);
    const int pair_ok = (a.ld_out % 2 == 0) && mmf_aligned(a.out, (size_t)2 * es) && (a.N / a.groups) % 2 == 0 ? 1 : 0;
    const int sms = g_num_sms();
    const int n_group = a.N / a.groups;

    for (int m0 = 0; m0 < a.M; m0 += rows_per_block) {
        StreamParams p;
        p.KC = KC;
        p.m0 = m0;
        p.mb = a.M - m0 < rows_per_block ? a.M - m0 : rows_per_block;
        const int MT = p.mb <= 8 ? 1 : p.mb <= 16 ? 2 : p.mb <= 32 ? 4 : 8;
        p.slabs_per_group = (n_group + SK_SLAB_ROWS - 1) / SK_SLAB_ROWS;
        p.tiles_per_group = (n_group + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
        p.ctas_per_group = sms / a.groups < 1 ? 1 : sms / a.groups;
        if (p.ctas_per_group > p.slabs_per_group) p.ctas_per_group = p.slabs_per_group;
        const int max_j = (p.slabs_per_group + p.ctas_per_group - 1) / p.ctas_per_group;
        // Two slabs in flight when the CTA has more than one and shared memory allows; then as deep a ring as fits.
        // Kernels of a decode step start while their predecessors still run (programmatic dependent launch) and use
        // that time to fetch their weights, which only works if both fit on an SM side by side: stay under ~108 KB
        // when the minimum configuration allows it, otherwise take what a single CTA may have.
        p.SL = max_j >= 2 && stream_smem(KC, MT, 2, 1) <= SK_SMEM_MAX ? 2 : 1;
        const size_t budget = stream_smem(KC, MT, p.SL, 1) <= 108 * 1024 ? 108 * 1024 : SK_SMEM_MAX;
        int depth = 1;
        const int max_depth = (max_j + p.SL - 1) / p.SL;
        while (depth < max_depth && p.SL * (depth + 1) <= SK_MAX_SLOTS && stream_smem(KC, MT, p.SL, depth + 1) <= budget) ++depth;
        p.depth = depth;
        const size_t smem = stream_smem(KC, MT, p.SL, depth);
        MMF_REQUIRE(smem <= SK_SMEM_MAX, MMF_ERR_BAD_SHAPE, "mmf_bitlinear_decode: shared memory budget exceeded (K=%d)", a.K);
        const dim3 grid((unsigned)(p.ctas_per_group * a.groups));
        const uint8_t* sl8 = static_cast<const uint8_t*>(slabs);
        switch (MT) {
            case 1: MMF_CUDA(mmf_launch_pdl(bitlinear_stream_kernel<1>, grid, dim3(SK_THREADS), smem, st, a, sl8, p, pair_ok)); break;
            case 2: MMF_CUDA(mmf_launch_pdl(bitlinear_stream_kernel<2>, grid, dim3(SK_THREADS), smem, st, a, sl8, p, pair_ok)); break;
            case 4: MMF_CUDA(mmf_launch_pdl(bitlinear_stream_kernel<4>, grid, dim3(SK_THREADS), smem, st, a, sl8, p, pair_ok)); break;
            default: MMF_CUDA(mmf_launch_pdl(bitlinear_stream_kernel<8>, grid, dim3(SK_THREADS), smem, st, a, sl8, p, pair_ok)); break;
        }
        MMF_LAUNCH_CHECK("bitlinear_stream_kernel");
    }
    return MMF_OK;
}

extern "C" int mmf_bitlinear_decode(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed_slabs,
                                    const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                                    int32_t* acc_out, int64_t M, int64_t N, int64_t K, int32_t* status, void* stream) {
    MMF_REQUIRE(q && dq && rowsum && packed_slabs && w_scale && out, MMF_ERR_BAD_ARG, "mmf_bitlinear_decode: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(out_dtype), MMF_ERR_BAD_ARG, "mmf_bitlinear_decode: unknown dtype %d", out_dtype);
    MMF_REQUIRE(M >= 0 && N > 0 && K > 0 && K % MMF_TILE_K == 0 && N < (1ll << 31) && K <= 65536, MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear_decode: need K %% 64 == 0 (M=%lld N=%lld K=%lld)", (long long)M, (long long)N, (long long)K);
    MMF_REQUIRE(M <= MMF_STREAM_MAX_M, MMF_ERR_BAD_SHAPE, "mmf_bitlinear_decode: M=%lld exceeds %d token rows; use mmf_bitlinear",
                (long long)M, MMF_STREAM_MAX_M);
    MMF_REQUIRE(groups >= 1 && N % groups == 0 && (groups == 1 || (N / groups) % MMF_TILE_ROWS == 0), MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear_decode: N/groups must be a multiple of 128 when groups > 1");
    MMF_REQUIRE(ld_out >= N, MMF_ERR_BAD_SHAPE, "mmf_bitlinear_decode: ld_out < N");
    MMF_REQUIRE(mmf_aligned(q, 16) && mmf_aligned(packed_slabs, 16), MMF_ERR_ALIGN,
                "mmf_bitlinear_decode: q and packed_slabs must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    BitLinearArgs a;
    a.q = q; a.dq = dq; a.rowsum = rowsum; a.packed = nullptr; a.w_scale = w_scale;
    a.out = out; a.acc_out = acc_out; a.out_dtype = out_dtype; a.ld_out = ld_out;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.groups = groups;
    a.ws = status; a.ws_bytes = status ? 4 : 0;
    return bitlinear_stream_launch(a, packed_slabs, (cudaStream_t)stream);
}
#endif  // MMF_EXPERIMENTS
