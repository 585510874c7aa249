// BitLinear for a handful of token rows (decode): a weight-streaming GEMV on the integer
// dot-product units.
//
// Two kernels live here.  bitlinear_gemv_rows_kernel (default) reduces over K inside the CTA; the older
// bitlinear_gemv_kernel splits K ACROSS CTAs through an int32 workspace — it remains for shapes whose
// activation rows do not fit in shared memory and behind mmf_bitlinear_gemv_static.
//
// The contraction is HBM-bound on the 2-bit weight stream (K*N/4 bytes; activations are a
// few KB and live in shared memory).  One CTA = one 128-row weight tile x one slice of K;
// thread r owns output row r, so each 16-byte load of a warp is one fully used 512-byte run
// of the tile-major weight buffer.  A 32-bit word carries 16 weights as (code+1) fields laid
// out so that (word >> 2i) & 0x03030303 is four consecutive columns as bytes -> one dp4a per
// 4 weights per token row; the +1 bias is removed with the per-row code sum in the epilogue.
// K is split across CTAs so that about two waves of CTAs cover the GPU even for a
// 2048x2048 layer (1 MB of weights); partial sums meet in an int32 workspace with atomics
// (integer adds commute, so the result is deterministic) and the last CTA of a tile runs
// the epilogue and zeroes the workspace again.
#include <mutex>

#include "bitlinear.cuh"

namespace {

constexpr int GV_THREADS = MMF_TILE_ROWS;  // 128

template <int MB>
__global__ void __launch_bounds__(GV_THREADS)
bitlinear_gemv_kernel(BitLinearArgs a, int KC, int kc_per_cta, int ksplit, int n_tiles, int group_tiles) {
    extern __shared__ __align__(16) int8_t xs[];  // [MB][kc_per_cta*64]
    __shared__ int s_last;
    pdl_trigger();
    const int ks = blockIdx.x, tile = blockIdx.y, mblk = blockIdx.z;
    const int r = threadIdx.x;
    const int m0 = mblk * MB;
    const int g = tile / group_tiles;
    const int kc0 = ks * kc_per_cta;
    const int kc1 = min(KC, kc0 + kc_per_cta);
    const int kslice = (kc1 - kc0) * MMF_TILE_K;  // bytes of activation codes per row in this CTA
    const int row_stride = kc_per_cta * MMF_TILE_K;

    // the first weight pieces do not depend on the preceding kernel: request them before the dependency wait
    const uint4* wp = a.packed + ((int64_t)tile * KC + kc0) * MMF_TILE_ROWS + r;
    const int nkc = kc1 - kc0;
    uint4 w_first[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w_first[i] = i < nkc ? __ldg(wp + (int64_t)i * MMF_TILE_ROWS) : make_uint4(0, 0, 0, 0);
    pdl_wait();

    // stage the activation codes of this K slice (16-byte pieces)
    const int8_t* qg = a.q + ((int64_t)g * a.M) * a.K + (int64_t)kc0 * MMF_TILE_K;
    const int pieces_per_row = kslice / 16;
    for (int p = r; p < MB * pieces_per_row; p += GV_THREADS) {
        const int m = p / pieces_per_row, off = (p % pieces_per_row) * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m0 + m < a.M) v = *reinterpret_cast<const uint4*>(qg + (int64_t)(m0 + m) * a.K + off);
        *reinterpret_cast<uint4*>(xs + m * row_stride + off) = v;
    }
    __syncthreads();

    int acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0;

    auto consume = [&](const uint4& wv, int kc) {
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) b[i] = (words[qd] >> (2 * i)) & 0x03030303u;
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const int4 xv = *reinterpret_cast<const int4*>(xs + m * row_stride + kc * MMF_TILE_K + qd * 16);
                acc[m] = __dp4a((int)b[0], xv.x, acc[m]);
                acc[m] = __dp4a((int)b[1], xv.y, acc[m]);
                acc[m] = __dp4a((int)b[2], xv.z, acc[m]);
                acc[m] = __dp4a((int)b[3], xv.w, acc[m]);
            }
        }
    };
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i < nkc) consume(w_first[i], i);
#pragma unroll 4
    for (int kc = 4; kc < nkc; ++kc) consume(__ldg(wp + (int64_t)kc * MMF_TILE_ROWS), kc);

    const int n = tile * MMF_TILE_ROWS + r;
    const int Npad = n_tiles * MMF_TILE_ROWS;
    bool do_epilogue = true;
    if (ksplit > 1) {
        uint32_t* cnt = reinterpret_cast<uint32_t*>(a.ws) + MMF_WS_HEADER + tile * MMF_WS_MBLK + mblk;
        int32_t* wacc = a.ws + MMF_WS_HEADER + (int64_t)n_tiles * MMF_WS_MBLK;
#pragma unroll
        for (int m = 0; m < MB; ++m)
            if (m0 + m < a.M) atomicAdd(wacc + (int64_t)(m0 + m) * Npad + n, acc[m]);
        __threadfence();
        __syncthreads();
        if (r == 0) s_last = (atomicAdd(cnt, 1u) == (uint32_t)(ksplit - 1));
        __syncthreads();
        do_epilogue = s_last;
        if (do_epilogue) {
            __threadfence();
#pragma unroll
            for (int m = 0; m < MB; ++m)
                if (m0 + m < a.M) {
                    int32_t* p = wacc + (int64_t)(m0 + m) * Npad + n;
                    acc[m] = __ldcg(p);
                    __stcg(p, 0);
                }
            if (r == 0) *cnt = 0u;
        }
    }
    if (do_epilogue && n < a.N) {
        const float wsc = a.w_scale[g];
#pragma unroll
        for (int m = 0; m < MB; ++m) {
            const int mm = m0 + m;
            if (mm < a.M) {
                const int64_t gm = (int64_t)g * a.M + mm;
                const int32_t v = acc[m] - a.rowsum[gm];
                if (a.acc_out) a.acc_out[(int64_t)mm * a.N + n] = v;
                store_out(a.out, a.out_dtype, (int64_t)mm * a.ld_out + n, bitlinear_dequant(v, a.dq[gm], wsc));
            }
        }
    }
}

// -----------------------------------------------------------------------------------------------------------
// Variant without any cross-CTA reduction (the default): one CTA = 32 rows of a weight tile x all of K.
// Warp w owns a 1/16 slice of K, lane l owns row l of the 32-row slice, so a warp's 16-byte loads are one
// 512-byte run of the tile-major buffer; the 16 partial sums per output meet in shared memory.  With 4 CTAs per
// weight tile even a 2048 x 2048 layer is spread over 64 CTAs and every thread has all its weight loads in
// flight at once; the first of them are requested before the grid-dependency wait.
// -----------------------------------------------------------------------------------------------------------
constexpr int G2_WARPS = 16;
constexpr int G2_THREADS = G2_WARPS * 32;
constexpr int G2_PF = 6;   // weight vectors requested before the dependency wait

template <int MB>
__global__ void __launch_bounds__(G2_THREADS)
bitlinear_gemv_rows_kernel(BitLinearArgs a, int KC, int group_tiles) {
    extern __shared__ __align__(16) int8_t smem2[];
    int8_t* xs = smem2;                                                  // [MB][K] activation codes
    int* red = reinterpret_cast<int*>(smem2 + (size_t)MB * a.K);         // [G2_WARPS][MB][32]
    pdl_trigger();
    const int tile = blockIdx.x >> 2, rq = blockIdx.x & 3, mblk = blockIdx.y;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = mblk * MB;
    const int g = tile / group_tiles;
    const int cpw = (KC + G2_WARPS - 1) / G2_WARPS;
    const int kc0 = min(KC, w * cpw), kc1 = min(KC, kc0 + cpw);
    const int nkc = kc1 - kc0;
    const uint4* wp = a.packed + ((int64_t)tile * KC + kc0) * MMF_TILE_ROWS + rq * 32 + lane;
    uint4 wf[G2_PF];
#pragma unroll
    for (int i = 0; i < G2_PF; ++i) wf[i] = i < nkc ? __ldg(wp + (int64_t)i * MMF_TILE_ROWS) : make_uint4(0, 0, 0, 0);
    pdl_wait();

    const int8_t* qg = a.q + ((int64_t)g * a.M) * a.K;
    const int pieces_per_row = a.K / 16;
    for (int p = threadIdx.x; p < MB * pieces_per_row; p += G2_THREADS) {
        const int m = p / pieces_per_row, off = (p - m * pieces_per_row) * 16;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (m0 + m < a.M) v = *reinterpret_cast<const uint4*>(qg + (int64_t)(m0 + m) * a.K + off);
        *reinterpret_cast<uint4*>(xs + (size_t)m * a.K + off) = v;
    }
    __syncthreads();

    int acc[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[m] = 0;
    auto consume = [&](const uint4& wv, int kc) {
        const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) b[i] = (words[qd] >> (2 * i)) & 0x03030303u;
#pragma unroll
            for (int m = 0; m < MB; ++m) {
                const int4 xv = *reinterpret_cast<const int4*>(xs + (size_t)m * a.K + (size_t)(kc0 + kc) * MMF_TILE_K + qd * 16);
                acc[m] = __dp4a((int)b[0], xv.x, acc[m]);
                acc[m] = __dp4a((int)b[1], xv.y, acc[m]);
                acc[m] = __dp4a((int)b[2], xv.z, acc[m]);
                acc[m] = __dp4a((int)b[3], xv.w, acc[m]);
            }
        }
    };
#pragma unroll
    for (int i = 0; i < G2_PF; ++i)
        if (i < nkc) consume(wf[i], i);
#pragma unroll 4
    for (int kc = G2_PF; kc < nkc; ++kc) consume(__ldg(wp + (int64_t)kc * MMF_TILE_ROWS), kc);

#pragma unroll
    for (int m = 0; m < MB; ++m) red[(w * MB + m) * 32 + lane] = acc[m];
    __syncthreads();
    if (threadIdx.x < MB * 32) {
        const int m = threadIdx.x >> 5, r = threadIdx.x & 31;
        int v = 0;
#pragma unroll
        for (int ww = 0; ww < G2_WARPS; ++ww) v += red[(ww * MB + m) * 32 + r];
        const int n = tile * MMF_TILE_ROWS + rq * 32 + r;
        const int mm = m0 + m;
        if (n < a.N && mm < a.M) {
            const int64_t gm = (int64_t)g * a.M + mm;
            v -= a.rowsum[gm];
            if (a.acc_out) a.acc_out[(int64_t)mm * a.N + n] = v;
            store_out(a.out, a.out_dtype, (int64_t)mm * a.ld_out + n, bitlinear_dequant(v, a.dq[gm], a.w_scale[g]));
        }
    }
}

}  // namespace

int bitlinear_gemv_launch(const BitLinearArgs& a, cudaStream_t st, bool force_split_k) {
    const int KC = a.K / MMF_TILE_K;
    const int n_tiles = (a.N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const int group_tiles = n_tiles / a.groups;
    const int MB = a.M <= 1 ? 1 : a.M <= 2 ? 2 : a.M <= 4 ? 4 : 8;
    const int mblocks = (a.M + MB - 1) / MB;
    MMF_REQUIRE(mblocks <= 65535, MMF_ERR_BAD_SHAPE, "mmf_bitlinear(gemv): M too large for the GEMV kernel");
    const size_t smem_rows = (size_t)MB * a.K + (size_t)G2_WARPS * MB * 32 * sizeof(int);
    if (!force_split_k && smem_rows <= 160 * 1024) {
        const dim3 grid2((unsigned)(n_tiles * 4), (unsigned)mblocks);
#define G2_LAUNCH(MBV)                                                                                              \
    {                                                                                                               \
        auto kfn = bitlinear_gemv_rows_kernel<MBV>;                                                                 \
        if (smem_rows > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows)); \
        MMF_CUDA(mmf_launch_pdl(kfn, grid2, dim3(G2_THREADS), smem_rows, st, a, KC, group_tiles));                 \
    }
        switch (MB) {
            case 1: G2_LAUNCH(1); break;
            case 2: G2_LAUNCH(2); break;
            case 4: G2_LAUNCH(4); break;
            default: G2_LAUNCH(8); break;
        }
#undef G2_LAUNCH
        MMF_LAUNCH_CHECK("bitlinear_gemv_rows_kernel");
        return MMF_OK;
    }
    int ksplit = 1;
    const int64_t need_words = MMF_WS_HEADER + (int64_t)n_tiles * MMF_WS_MBLK + (int64_t)a.M * n_tiles * MMF_TILE_ROWS;
    const bool can_split = a.ws && a.M <= MMF_SPLITK_MAX_M && mblocks <= MMF_WS_MBLK && a.ws_bytes >= need_words * 4;
    if (can_split) {
        const int64_t base = (int64_t)n_tiles * mblocks;
        const int64_t target = 2 * 148;
        if (base < target) ksplit = (int)((target + base - 1) / base);
        if (ksplit > KC) ksplit = KC;
    }
    // shared memory holds MB rows of the K slice: cap the slice at 32 KB per row block
    int kc_per_cta = (KC + ksplit - 1) / ksplit;
    const int max_kc = (96 * 1024) / (MB * MMF_TILE_K);
    if (kc_per_cta > max_kc) {
        MMF_REQUIRE(can_split, MMF_ERR_WORKSPACE,
                    "mmf_bitlinear(gemv): K=%d needs split-K for %d rows per block; workspace missing or too small", a.K, MB);
        kc_per_cta = max_kc;
    }
    ksplit = (KC + kc_per_cta - 1) / kc_per_cta;
    const size_t smem = (size_t)MB * kc_per_cta * MMF_TILE_K;
    const dim3 grid((unsigned)ksplit, (unsigned)n_tiles, (unsigned)mblocks);
    MMF_REQUIRE(mblocks <= 65535, MMF_ERR_BAD_SHAPE, "mmf_bitlinear(gemv): M too large for the GEMV kernel");
#define GV_LAUNCH(MBV)                                                                                              \
    {                                                                                                               \
        auto kfn = bitlinear_gemv_kernel<MBV>;                                                                      \
        if (smem > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MMF_CUDA(mmf_launch_pdl(kfn, grid, dim3(GV_THREADS), smem, st, a, KC, kc_per_cta, ksplit, n_tiles, group_tiles)); \
    }
    switch (MB) {
        case 1: GV_LAUNCH(1); break;
        case 2: GV_LAUNCH(2); break;
        case 4: GV_LAUNCH(4); break;
        default: GV_LAUNCH(8); break;
    }
#undef GV_LAUNCH
    MMF_LAUNCH_CHECK("bitlinear_gemv_kernel");
    return MMF_OK;
}

extern "C" int64_t mmf_bitlinear_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const int64_t n_tiles = (N + MMF_TILE_ROWS - 1) / MMF_TILE_ROWS;
    const int64_t rows = M < MMF_SPLITK_MAX_M ? M : MMF_SPLITK_MAX_M;
    const int64_t words = MMF_WS_HEADER + n_tiles * MMF_WS_MBLK + rows * n_tiles * MMF_TILE_ROWS;
    return ((words * 4 + 255) / 256) * 256;
}

extern "C" int mmf_bitlinear(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed,
                             const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                             int32_t* acc_out, int64_t M, int64_t N, int64_t K, void* workspace,
                             int64_t workspace_bytes, int kernel, void* stream) {
    MMF_REQUIRE(q && dq && rowsum && packed && w_scale && out, MMF_ERR_BAD_ARG, "mmf_bitlinear: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(out_dtype), MMF_ERR_BAD_ARG, "mmf_bitlinear: unknown dtype %d", out_dtype);
    MMF_REQUIRE(M >= 0 && N > 0 && K > 0 && K % MMF_TILE_K == 0 && M < (1ll << 31) && N < (1ll << 31) && K <= 65536,
                MMF_ERR_BAD_SHAPE, "mmf_bitlinear: need K %% 64 == 0 (M=%lld N=%lld K=%lld)", (long long)M, (long long)N,
                (long long)K);
    MMF_REQUIRE(groups >= 1 && N % groups == 0 && (groups == 1 || (N / groups) % MMF_TILE_ROWS == 0), MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear: N/groups must be a multiple of 128 when groups > 1");
    MMF_REQUIRE(ld_out >= N, MMF_ERR_BAD_SHAPE, "mmf_bitlinear: ld_out < N");
    MMF_REQUIRE(mmf_aligned(q, 16) && mmf_aligned(packed, 16), MMF_ERR_ALIGN,
                "mmf_bitlinear: q and packed must be 16-byte aligned");
    MMF_REQUIRE(!workspace || mmf_aligned(workspace, 16), MMF_ERR_ALIGN, "mmf_bitlinear: workspace must be 16-byte aligned");
    MMF_REQUIRE(kernel == MMF_KERNEL_AUTO || kernel == MMF_KERNEL_GEMV || kernel == MMF_KERNEL_MMA, MMF_ERR_BAD_ARG,
                "mmf_bitlinear: unknown kernel selector %d", kernel);
    if (M == 0) return MMF_OK;
    BitLinearArgs a;
    a.q = q; a.dq = dq; a.rowsum = rowsum; a.packed = (const uint4*)packed; a.w_scale = w_scale;
    a.out = out; a.acc_out = acc_out; a.out_dtype = out_dtype; a.ld_out = ld_out;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.groups = groups;
    a.ws = (int32_t*)workspace; a.ws_bytes = workspace ? workspace_bytes : 0;
    cudaStream_t st = (cudaStream_t)stream;
    const bool use_mma = kernel == MMF_KERNEL_MMA || (kernel == MMF_KERNEL_AUTO && M >= MMF_MMA_MIN_M);
    return use_mma ? bitlinear_mma_launch(a, st) : bitlinear_gemv_launch(a, st, false);
}

// =========================================================================================================
// Allocation-free variant of the small-batch BitLinear
// =========================================================================================================
// Split-K scratch that lives in the library image instead of in caller memory.  Every GPU that loads the
// library carries these MMF_STATIC_SCRATCH_BYTES until the process exits.
static __device__ __align__(256) int32_t g_gemv_scratch[MMF_STATIC_SCRATCH_BYTES / 4];

// Device address of g_gemv_scratch on the CURRENT device.  In host code the symbol's name is only a handle;
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device
// current and remembered.
static int gemv_static_scratch(int32_t** out) {
    static std::mutex mu;
    static int32_t* per_device[64] = {nullptr};
    int dev = -1;
    MMF_CUDA(cudaGetDevice(&dev));
    MMF_REQUIRE(dev >= 0 && dev < 64, MMF_ERR_CUDA, "mmf_bitlinear_gemv_static: unexpected device index %d", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!per_device[dev]) {
        void* p = nullptr;
        MMF_CUDA(cudaGetSymbolAddress(&p, g_gemv_scratch));
        MMF_REQUIRE(p != nullptr, MMF_ERR_CUDA, "mmf_bitlinear_gemv_static: cudaGetSymbolAddress returned no address");
        per_device[dev] = static_cast<int32_t*>(p);
    }
    *out = per_device[dev];
    return MMF_OK;
}

extern "C" int mmf_bitlinear_gemv_static(const int8_t* q, const float* dq, const int32_t* rowsum, const void* packed,
                                         const float* w_scale, int groups, void* out, int out_dtype, int64_t ld_out,
                                         int64_t M, int64_t N, int64_t K, void* stream) {
    MMF_REQUIRE(q && dq && rowsum && packed && w_scale && out, MMF_ERR_BAD_ARG, "mmf_bitlinear_gemv_static: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(out_dtype), MMF_ERR_BAD_ARG, "mmf_bitlinear_gemv_static: unknown dtype %d", out_dtype);
    MMF_REQUIRE(M >= 0 && N > 0 && K > 0 && K % MMF_TILE_K == 0 && M < (1ll << 31) && N < (1ll << 31) && K <= 65536,
                MMF_ERR_BAD_SHAPE, "mmf_bitlinear_gemv_static: need K %% 64 == 0 (M=%lld N=%lld K=%lld)", (long long)M,
                (long long)N, (long long)K);
    MMF_REQUIRE(groups >= 1 && N % groups == 0 && (groups == 1 || (N / groups) % MMF_TILE_ROWS == 0), MMF_ERR_BAD_SHAPE,
                "mmf_bitlinear_gemv_static: N/groups must be a multiple of 128 when groups > 1");
    MMF_REQUIRE(ld_out >= N, MMF_ERR_BAD_SHAPE, "mmf_bitlinear_gemv_static: ld_out < N");
    MMF_REQUIRE(mmf_aligned(q, 16) && mmf_aligned(packed, 16), MMF_ERR_ALIGN,
                "mmf_bitlinear_gemv_static: q and packed must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    const int64_t need = mmf_bitlinear_workspace_bytes(M, N, K);
    MMF_REQUIRE(need <= MMF_STATIC_SCRATCH_BYTES, MMF_ERR_WORKSPACE,
                "mmf_bitlinear_gemv_static: M=%lld N=%lld needs %lld bytes of split-K scratch but the built-in array holds "
                "%d; use mmf_bitlinear with a workspace of your own for this size",
                (long long)M, (long long)N, (long long)need, MMF_STATIC_SCRATCH_BYTES);
    int32_t* scratch = nullptr;
    const int rc = gemv_static_scratch(&scratch);
    if (rc != MMF_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // the array still holds whatever the last call left: zero the part this call accumulates into
    MMF_CUDA(cudaMemsetAsync(scratch, 0, (size_t)need, st));
    BitLinearArgs a;
    a.q = q; a.dq = dq; a.rowsum = rowsum; a.packed = (const uint4*)packed; a.w_scale = w_scale;
    a.out = out; a.acc_out = nullptr; a.out_dtype = out_dtype; a.ld_out = ld_out;
    a.M = (int)M; a.N = (int)N; a.K = (int)K; a.groups = groups;
    a.ws = scratch; a.ws_bytes = MMF_STATIC_SCRATCH_BYTES;
    return bitlinear_gemv_launch(a, st, /*force_split_k=*/true);   // the split-K kernel is the one that needs scratch
}
