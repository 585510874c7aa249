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
// Warp roles (224 threads): warps 0-3 unpack (thread t <-> TMEM lane t <-> weight row t) and
// later run the epilogue; warp 4 = activation-tile TMA producer; warp 5 = TMEM owner + MMA
// issuer; warp 6 = packed-weight TMA producer.  Three rings (packed weights in smem, unpacked
// A chunks in TMEM, activation tiles in smem) are synchronised with mbarriers; every wait is
// bounded and reports through a status word instead of hanging.
//
// Weights are stored biased (+1); sum_k (t+1)*x = acc + rowsum(x) and the epilogue subtracts the
// per-token code sum.  For few tokens the K range is split over the CTAs of a thread-block cluster
// (2, 4 or 8) to fill the GPU; each CTA parks its partial int32 tile in its own shared memory and,
// after a cluster barrier, reduces its share of the token columns over its peers' tiles through
// distributed shared memory (integer adds: deterministic) and dequantises them.
#include <cuda.h>

#include "bitlinear.cuh"

namespace {

constexpr int MM_THREADS = 224;
constexpr int SA = 8;             // A chunks (64 K each, 16 TMEM columns) in flight
constexpr int SB = 4;             // activation stages (128 K each)
constexpr int SW = 12;            // packed-weight stages (128 K = 4 KB each)
constexpr int W_STAGE_BYTES = 2 * MMF_TILE_ROWS * 16;  // two 64-K chunks
constexpr long long WAIT_LIMIT_CYCLES = 2000000000ll;

struct MmaParams {
    int KC;              // K / 64
    int n_tiles, group_tiles;
    int NT;              // token rows per tile (multiple of 16, <= 256)
    int ksplit;          // CTAs sharing one output tile along K
    int stages_per_cta;  // 128-K stages per CTA
    int tmem_cols;       // power of two >= NT + SA*16
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
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
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
__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ int32_t ld_peer_s32(const void* my_smem, uint32_t peer_rank) {
    uint32_t remote;
    int32_t v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem)), "r"(peer_rank));
    asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
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

struct __align__(8) Barriers {
    uint64_t b_full[SB], b_empty[SB];
    uint64_t w_full[SW], w_empty[SW];
    uint64_t a_full[SA], a_empty[SA];
    uint64_t acc_full;
};

__global__ void __launch_bounds__(MM_THREADS, 1)
bitlinear_mma_kernel(const __grid_constant__ CUtensorMap q_map, BitLinearArgs a, MmaParams p) {
    extern __shared__ uint8_t smem_raw[];
    // carve: [B ring | W ring] aligned to 1024 B (required by the 128-byte swizzle atoms)
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_stage_bytes = p.NT * 128;
    uint8_t* b_ring = base;
    uint8_t* w_ring = base + SB * b_stage_bytes;

    __shared__ Barriers bars;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ float s_dq[256];
    __shared__ int s_rs[256];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int ks = blockIdx.x, tile = blockIdx.y, mt = blockIdx.z;
    const int g = tile / p.group_tiles;
    const int m0 = mt * p.NT;
    const int stage0 = ks * p.stages_per_cta;
    const int total_stages = (p.KC + 1) / 2;
    const int nstages = min(p.stages_per_cta, total_stages - stage0);   // >= 1 by construction

    if (tid == 0) {
        for (int i = 0; i < SB; ++i) { mbar_init(&bars.b_full[i], 1); mbar_init(&bars.b_empty[i], 1); }
        for (int i = 0; i < SW; ++i) { mbar_init(&bars.w_full[i], 1); mbar_init(&bars.w_empty[i], 128); }
        for (int i = 0; i < SA; ++i) { mbar_init(&bars.a_full[i], 128); mbar_init(&bars.a_empty[i], 1); }
        mbar_init(&bars.acc_full, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < p.NT; i += MM_THREADS) {
        const int m = m0 + i;
        const bool ok = m < a.M;
        s_dq[i] = ok ? a.dq[(int64_t)g * a.M + m] : 0.0f;
        s_rs[i] = ok ? a.rowsum[(int64_t)g * a.M + m] : 0;
    }
    if (warp == 5) tmem_alloc(&s_tmem_base, (uint32_t)p.tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    const uint32_t tmem_a = tmem_base + (uint32_t)p.NT;   // A stages follow the accumulator columns
    volatile int* abort_flag = &s_abort;

    if (warp == 4) {
        // ------------------------------------------------------------ activation tiles (TMA, swizzled)
        if (elect_one()) {
            for (int i = 0; i < nstages; ++i) {
                const int s = i % SB;
                if (!mbar_wait(&bars.b_empty[s], ((i / SB) & 1) ^ 1, abort_flag)) break;
                mbar_expect_tx(&bars.b_full[s], (uint32_t)b_stage_bytes);
                tma_load_2d(b_ring + s * b_stage_bytes, &q_map, &bars.b_full[s], (stage0 + i) * 128, g * a.M + m0);
            }
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ packed weights (bulk TMA)
        if (elect_one()) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(a.packed) + ((int64_t)tile * p.KC) * (MMF_TILE_ROWS * 16);
            for (int i = 0; i < nstages; ++i) {
                const int s = i % SW;
                if (!mbar_wait(&bars.w_empty[s], ((i / SW) & 1) ^ 1, abort_flag)) break;
                const int kc = (stage0 + i) * 2;
                const uint32_t bytes = (uint32_t)min(2, p.KC - kc) * (MMF_TILE_ROWS * 16);
                mbar_expect_tx(&bars.w_full[s], bytes);
                bulk_load_1d(w_ring + s * W_STAGE_BYTES, src + (int64_t)kc * (MMF_TILE_ROWS * 16), bytes, &bars.w_full[s]);
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issue
        if (elect_one()) {
            int ac = 0;  // running A-chunk counter
            bool ok = true;
            for (int i = 0; i < nstages && ok; ++i) {
                const int s = i % SB;
                ok = mbar_wait(&bars.b_full[s], (i / SB) & 1, abort_flag);
                if (!ok) break;
                const uint32_t b_addr = smem_u32(b_ring + s * b_stage_bytes);
                const int nch = min(2, p.KC - (stage0 + i) * 2);
                for (int h = 0; h < nch; ++h, ++ac) {
                    const int as = ac % SA;
                    ok = mbar_wait(&bars.a_full[as], (ac / SA) & 1, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const uint64_t bd = make_b_desc(b_addr + h * 64 + j * 32);
                        mma_i8_ts(tmem_base, tmem_a + as * 16 + j * 8, bd, p.idesc, (ac | j) != 0 ? 1u : 0u);
                    }
                    tc_commit(&bars.a_empty[as]);   // frees the A chunk when these MMAs retire
                }
                tc_commit(&bars.b_empty[s]);
            }
            tc_commit(&bars.acc_full);
        }
    } else {
        // ------------------------------------------------------------ unpack (warps 0-3), then epilogue
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        int ac = 0;
        bool ok = true;
        for (int i = 0; i < nstages && ok; ++i) {
            const int s = i % SW;
            ok = __all_sync(0xffffffffu, mbar_wait(&bars.w_full[s], (i / SW) & 1, abort_flag));   // warp-uniform
            if (!ok) break;
            const int nch = min(2, p.KC - (stage0 + i) * 2);
            for (int h = 0; h < nch; ++h, ++ac) {
                const uint4 wv = *reinterpret_cast<const uint4*>(w_ring + s * W_STAGE_BYTES + h * (MMF_TILE_ROWS * 16) + tid * 16);
                const int as = ac % SA;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars.a_empty[as], ((ac / SA) & 1) ^ 1, abort_flag));
                if (!ok) break;   // uniform per warp: the .sync.aligned tcgen05 ops below need the whole warp
                const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                uint32_t r[16];
#pragma unroll
                for (int qd = 0; qd < 4; ++qd)
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) r[qd * 4 + k4] = (words[qd] >> (2 * k4)) & 0x03030303u;
                tmem_st16(tmem_a + lane_addr + as * 16, r);
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&bars.a_full[as]);
            }
            mbar_arrive(&bars.w_empty[s]);
        }

        // epilogue: thread <-> weight row n, columns <-> tokens
        ok = __all_sync(0xffffffffu, ok && mbar_wait(&bars.acc_full, 0, abort_flag));
        tc_fence_after();
        if (ok) {
            const int n = tile * MMF_TILE_ROWS + tid;
            const float wsc = a.w_scale[g];
            int32_t* part = reinterpret_cast<int32_t*>(b_ring);   // [NT][128] partial tile (the ring is idle now)
            for (int c0 = 0; c0 < p.NT; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(tmem_base + lane_addr + c0, v);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    if (p.ksplit > 1) {
                        part[(c0 + j) * MMF_TILE_ROWS + tid] = (int32_t)v[j];
                    } else {
                        const int m = m0 + c0 + j;
                        if (m < a.M && n < a.N) {
                            const int32_t acc = (int32_t)v[j] - s_rs[c0 + j];
                            if (a.acc_out) a.acc_out[(int64_t)m * a.N + n] = acc;
                            store_out(a.out, a.out_dtype, (int64_t)m * a.ld_out + n, bitlinear_dequant(acc, s_dq[c0 + j], wsc));
                        }
                    }
                }
            }
        }
    }

    if (p.ksplit > 1) {
        // split-K: every CTA of the cluster has parked its partial tile; reduce my share of the token columns
        cluster_sync_all();
        if (warp < 4 && !*abort_flag) {
            const int n = tile * MMF_TILE_ROWS + tid;
            const float wsc = a.w_scale[g];
            const int32_t* part = reinterpret_cast<const int32_t*>(b_ring);
            const int per = p.NT / p.ksplit;
            for (int c = ks * per; c < (ks + 1) * per; ++c) {
                int32_t acc = 0;
                for (int peer = 0; peer < p.ksplit; ++peer) acc += ld_peer_s32(part + c * MMF_TILE_ROWS + tid, (uint32_t)peer);
                const int m = m0 + c;
                if (m < a.M && n < a.N) {
                    acc -= s_rs[c];
                    if (a.acc_out) a.acc_out[(int64_t)m * a.N + n] = acc;
                    store_out(a.out, a.out_dtype, (int64_t)m * a.ld_out + n, bitlinear_dequant(acc, s_dq[c], wsc));
                }
            }
        }
        cluster_sync_all();   // peers may still be reading this CTA's shared memory
    }

    // teardown: everyone meets, TMEM goes back; on the error path give copies in flight time to land first
    if (*abort_flag) {
        __nanosleep(20000);
        if (tid == 0 && a.ws) atomicExch(reinterpret_cast<int*>(a.ws), 1);   // status word: a wait gave up
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
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

int bitlinear_mma_launch(const BitLinearArgs& a, cudaStream_t st) {
    MmaParams p;
    p.KC = a.K / MMF_TILE_K;
    p.n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    p.group_tiles = p.n_tiles / a.groups;
    p.NT = a.M >= 256 ? 256 : ((a.M + 15) / 16) * 16;
    const int m_tiles = (a.M + p.NT - 1) / p.NT;
    const int total_stages = (p.KC + 1) / 2;
    // split K over a cluster of 2/4/8 CTAs until the grid covers the GPU
    p.ksplit = 1;
    while (p.ksplit < 8 && (int64_t)p.n_tiles * m_tiles * p.ksplit < 148 && p.ksplit * 2 <= total_stages) p.ksplit *= 2;
    p.stages_per_cta = (total_stages + p.ksplit - 1) / p.ksplit;
    while (p.ksplit > 1 && p.stages_per_cta * (p.ksplit - 1) >= total_stages) {   // every CTA must own >= 1 stage
        p.ksplit /= 2;
        p.stages_per_cta = (total_stages + p.ksplit - 1) / p.ksplit;
    }
    int cols = 32;
    while (cols < p.NT + SA * 16) cols *= 2;
    p.tmem_cols = cols;
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

    const size_t smem = 1024 + (size_t)SB * p.NT * 128 + (size_t)SW * W_STAGE_BYTES;
    MMF_CUDA(cudaFuncSetAttribute(bitlinear_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((unsigned)p.ksplit, (unsigned)p.n_tiles, (unsigned)m_tiles);
    MMF_REQUIRE(m_tiles <= 65535 && p.n_tiles <= 65535, MMF_ERR_BAD_SHAPE, "mmf_bitlinear(mma): problem too large");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(MM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)p.ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MMF_CUDA(cudaLaunchKernelEx(&cfg, bitlinear_mma_kernel, q_map, a, p));
    MMF_LAUNCH_CHECK("bitlinear_mma_kernel");
    return MMF_OK;
}
