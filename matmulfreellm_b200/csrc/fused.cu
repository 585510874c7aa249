// Fused row-wise kernels of the HGRNBit block: every tensor that sits between two BitLinear
// contractions is produced, normalised and re-quantised to int8 codes in one pass, so the only
// activations that touch HBM between contractions are the codes themselves.
//
// Rounding points follow the reference's op sequence: wherever the reference materialises a
// tensor in the activation dtype T (bf16/fp16/fp32) the value is rounded to T here too
// (round_to<T>), and all statistics are taken exactly where the reference takes them.
//
//   prenorm_quant : [x + residual] -> residual_out ; RMSNorm(block norm) -> T ; G x (BitLinear RMSNorm
//                   + int8 quant) sharing one row statistic        (attn_norm -> i/f/g, mlp_norm -> gate)
//   gatenorm_quant: RMSNorm(g) * w * o * sigmoid(o) -> T ; BitLinear RMSNorm + quant   (g_norm -> o_proj)
//   swiglu_quant  : silu(gate) * up -> T ; BitLinear RMSNorm + quant                   (MLP -> down_proj)
// (the gate math of the recurrence itself is fused into the scan kernel, hgrn.cu)
#include "common.cuh"

namespace {

constexpr int FT = 256;  // threads per row CTA

__device__ __forceinline__ void block_max3(float (&v)[3], float* red /* >= 3*33 */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int k = 0; k < 3; ++k) v[k] = warp_max(v[k]);
    __syncthreads();
    if (lane == 0) { red[wid] = v[0]; red[33 + wid] = v[1]; red[66 + wid] = v[2]; }
    __syncthreads();
    if (wid == 0) {
#pragma unroll
        for (int k = 0; k < 3; ++k) {
            float t = lane < nw ? red[33 * k + lane] : 0.0f;
            t = warp_max(t);
            if (lane == 0) red[33 * k + 32] = t;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 3; ++k) v[k] = red[33 * k + 32];
}

// quantise the row cached in `row` (already = y1, the BitLinear's input in T precision) for projection g
template <int V>
__device__ __forceinline__ void quant_store(const float* row, int D, float rstd, const float* nw, float s,
                                            int8_t* qr, int& lsum) {
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        int8_t codes[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float y = __fmul_rn(row[c + i], rstd);
            if (nw) y = __fmul_rn(y, nw[c + i]);
            float r = rintf(__fmul_rn(y, s));
            r = fminf(fmaxf(r, -128.0f), 127.0f);
            const int iv = (int)r;
            codes[i] = (int8_t)iv;
            lsum += iv;
        }
        if constexpr (V == 8) *reinterpret_cast<uint2*>(qr + c) = *reinterpret_cast<const uint2*>(codes);
        else *reinterpret_cast<uint32_t*>(qr + c) = *reinterpret_cast<const uint32_t*>(codes);
    }
}

// BitLinear prologue on a row already cached in shared memory as T-precision floats:
// one shared sum of squares, then per projection absmax -> scale -> codes.
template <int V, int G>
__device__ __forceinline__ void bitlinear_prologue(float* row, int D, double ss, float eps, const float* const* nws,
                                                   int8_t* const* qs, float* const* dqs, int32_t* const* rss, int64_t m,
                                                   double* redd, float* redf, int* redi) {
    const float rstd = rstd_from_sumsq(block_sum(ss, redd), D, eps);
    float amax[3] = {0.0f, 0.0f, 0.0f};
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float y = __fmul_rn(row[c + i], rstd);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float yg = nws[g] ? __fmul_rn(y, nws[g][c + i]) : y;
                amax[g] = fmaxf(amax[g], fabsf(yg));
            }
        }
    }
    block_max3(amax, redf);
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float a = fmaxf(amax[g], 1e-5f);
        const float s = __fdiv_rn(127.0f, a);
        int lsum = 0;
        quant_store<V>(row, D, rstd, nws[g], s, qs[g] + m * (int64_t)D, lsum);
        lsum = block_sum(lsum, redi);
        if (threadIdx.x == 0) {
            dqs[g][m] = __fdiv_rn(a, 127.0f);
            rss[g][m] = lsum;
        }
    }
}

struct PrenormArgs {
    const void* x; int64_t ld_x;
    const void* res; int64_t ld_res;      // may be null
    void* res_out;                         // [M, D] contiguous, may be null
    void* y_out;                           // [M, D] contiguous: the normed row in T, may be null
    const float* norm_w; float eps_norm;   // block-level RMSNorm
    const float* nws[3]; float eps_bl;     // per-projection BitLinear norm weights
    int8_t* q; float* dq; int32_t* rowsum; // [G][M][D], [G][M], [G][M]
    int64_t M; int D; int G;
    int round_sum_first;                   // 1: the reference added x+residual as a tensor op (rounded to T) before norm
};

template <typename T>
__global__ void __launch_bounds__(FT)
prenorm_quant_kernel(PrenormArgs a) {
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    __shared__ float redf[99];
    __shared__ int redi[33];
    constexpr int V = 16 / sizeof(T);
    const int64_t m = blockIdx.x;
    const int D = a.D;
    const T* xr = reinterpret_cast<const T*>(a.x) + m * a.ld_x;
    const T* rr = a.res ? reinterpret_cast<const T*>(a.res) + m * a.ld_res : nullptr;
    T* ro = a.res_out ? reinterpret_cast<T*>(a.res_out) + m * (int64_t)D : nullptr;

    double ss = 0.0;
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        float v[V];
        load16<T>(xr + c, v);
        if (rr) {
            float r[V];
            load16<T>(rr + c, r);
#pragma unroll
            for (int i = 0; i < V; ++i) v[i] = __fadd_rn(v[i], r[i]);
        }
        if (ro) store16<T>(ro + c, v);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            if (a.round_sum_first) v[i] = round_to<T>(v[i]);
            row[c + i] = v[i];
            ss += (double)v[i] * (double)v[i];
        }
    }
    const float rstd1 = rstd_from_sumsq(block_sum(ss, redd), D, a.eps_norm);
    T* yo = a.y_out ? reinterpret_cast<T*>(a.y_out) + m * (int64_t)D : nullptr;
    double ss2 = 0.0;
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float t = __fmul_rn(row[c + i], rstd1);
            if (a.norm_w) t = __fmul_rn(t, a.norm_w[c + i]);
            t = round_to<T>(t);
            o[i] = t;
            row[c + i] = t;
            ss2 += (double)t * (double)t;
        }
        if (yo) store16<T>(yo + c, o);
    }
    if (a.G == 0) return;
    const float* nws[3] = {a.nws[0], a.nws[1], a.nws[2]};
    int8_t* qs[3]; float* dqs[3]; int32_t* rss[3];
#pragma unroll
    for (int g = 0; g < 3; ++g) {
        qs[g] = a.q + (int64_t)g * a.M * D;
        dqs[g] = a.dq + (int64_t)g * a.M;
        rss[g] = a.rowsum + (int64_t)g * a.M;
    }
    if (a.G == 3) bitlinear_prologue<V, 3>(row, D, ss2, a.eps_bl, nws, qs, dqs, rss, m, redd, redf, redi);
    else bitlinear_prologue<V, 1>(row, D, ss2, a.eps_bl, nws, qs, dqs, rss, m, redd, redf, redi);
}

// y = round_T( ((g*rstd)*w) * o * sigmoid(o) ), then BitLinear prologue
template <typename T>
__global__ void __launch_bounds__(FT)
gatenorm_quant_kernel(const T* __restrict__ gx, int64_t ld_g, const T* __restrict__ o, int64_t ld_o,
                      const float* __restrict__ gw, float eps_g, const float* __restrict__ nw, float eps_bl,
                      int8_t* __restrict__ q, float* __restrict__ dq, int32_t* __restrict__ rowsum, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    __shared__ float redf[99];
    __shared__ int redi[33];
    constexpr int V = 16 / sizeof(T);
    const int64_t m = blockIdx.x;
    const T* gr = gx + m * ld_g;
    const T* orow = o + m * ld_o;
    double ss = 0.0;
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        float v[V];
        load16<T>(gr + c, v);
#pragma unroll
        for (int i = 0; i < V; ++i) { row[c + i] = v[i]; ss += (double)v[i] * (double)v[i]; }
    }
    const float rstd = rstd_from_sumsq(block_sum(ss, redd), D, eps_g);
    double ss2 = 0.0;
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        float ov[V];
        load16<T>(orow + c, ov);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float t = __fmul_rn(row[c + i], rstd);
            if (gw) t = __fmul_rn(t, gw[c + i]);
            t = __fmul_rn(t, ov[i]);
            t = round_to<T>(__fmul_rn(t, sigmoidf_(ov[i])));
            row[c + i] = t;
            ss2 += (double)t * (double)t;
        }
    }
    const float* nws[3] = {nw, nullptr, nullptr};
    int8_t* qs[3] = {q, nullptr, nullptr}; float* dqs[3] = {dq, nullptr, nullptr}; int32_t* rss[3] = {rowsum, nullptr, nullptr};
    bitlinear_prologue<V, 1>(row, D, ss2, eps_bl, nws, qs, dqs, rss, m, redd, redf, redi);
}

// z = round_T(silu(gate)*up), then BitLinear prologue.  gate/up are the two halves of a [M, 2D] tensor.
template <typename T>
__global__ void __launch_bounds__(FT)
swiglu_quant_kernel(const T* __restrict__ gate, const T* __restrict__ up, int64_t ld, const float* __restrict__ nw,
                    float eps_bl, int8_t* __restrict__ q, float* __restrict__ dq, int32_t* __restrict__ rowsum, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    __shared__ float redf[99];
    __shared__ int redi[33];
    constexpr int V = 16 / sizeof(T);
    const int64_t m = blockIdx.x;
    const T* gr = gate + m * ld;
    const T* ur = up + m * ld;
    double ss = 0.0;
    for (int c = threadIdx.x * V; c < D; c += FT * V) {
        float gv[V], uv[V];
        load16<T>(gr + c, gv);
        load16<T>(ur + c, uv);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float t = round_to<T>(silu_mul(gv[i], uv[i]));
            row[c + i] = t;
            ss += (double)t * (double)t;
        }
    }
    const float* nws[3] = {nw, nullptr, nullptr};
    int8_t* qs[3] = {q, nullptr, nullptr}; float* dqs[3] = {dq, nullptr, nullptr}; int32_t* rss[3] = {rowsum, nullptr, nullptr};
    bitlinear_prologue<V, 1>(row, D, ss, eps_bl, nws, qs, dqs, rss, m, redd, redf, redi);
}

}  // namespace

// =========================================================================================================
// C ABI
// =========================================================================================================
#define FUSED_ROW_CHECKS(name, D)                                                                                   \
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, name ": unknown dtype %d", dtype);                             \
    MMF_REQUIRE(M >= 0 && (D) > 0 && (D) <= 16384 && (D) % 16 == 0, MMF_ERR_BAD_SHAPE,                               \
                name ": need 0 < D <= 16384 and D %% 16 == 0 (D=%lld)", (long long)(D));

extern "C" int mmf_prenorm_quant(const void* x, int64_t ld_x, const void* residual, int64_t ld_res, int dtype,
                                 int round_sum_first, const float* norm_w, float eps_norm, void* residual_out,
                                 void* y_out, int groups, const float* nw0, const float* nw1, const float* nw2,
                                 float eps_bl, int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D,
                                 void* stream) {
    MMF_REQUIRE(x, MMF_ERR_BAD_ARG, "mmf_prenorm_quant: null x");
    FUSED_ROW_CHECKS("mmf_prenorm_quant", D);
    MMF_REQUIRE(groups == 0 || groups == 1 || groups == 3, MMF_ERR_BAD_ARG, "mmf_prenorm_quant: groups must be 0, 1 or 3");
    MMF_REQUIRE(groups == 0 || (q && dq && rowsum), MMF_ERR_BAD_ARG, "mmf_prenorm_quant: null output");
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(x, 16) && (ld_x * es) % 16 == 0 && (!residual || (mmf_aligned(residual, 16) && (ld_res * es) % 16 == 0)) &&
                    (!residual_out || mmf_aligned(residual_out, 16)) && (!y_out || mmf_aligned(y_out, 16)) && (!q || mmf_aligned(q, 16)),
                MMF_ERR_ALIGN, "mmf_prenorm_quant: rows must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    PrenormArgs a;
    a.x = x; a.ld_x = ld_x; a.res = residual; a.ld_res = ld_res; a.res_out = residual_out; a.y_out = y_out;
    a.norm_w = norm_w; a.eps_norm = eps_norm; a.nws[0] = nw0; a.nws[1] = nw1; a.nws[2] = nw2; a.eps_bl = eps_bl;
    a.q = q; a.dq = dq; a.rowsum = rowsum; a.M = M; a.D = (int)D; a.G = groups; a.round_sum_first = round_sum_first;
    const size_t smem = (size_t)D * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        if (smem > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(prenorm_quant_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        prenorm_quant_kernel<T><<<(unsigned)M, FT, smem, (cudaStream_t)stream>>>(a);
    });
    MMF_LAUNCH_CHECK("prenorm_quant_kernel");
    return MMF_OK;
}

extern "C" int mmf_gatenorm_quant(const void* g, int64_t ld_g, const void* o, int64_t ld_o, int dtype,
                                  const float* gnorm_w, float eps_g, const float* nw, float eps_bl, int8_t* q, float* dq,
                                  int32_t* rowsum, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(g && o && q && dq && rowsum, MMF_ERR_BAD_ARG, "mmf_gatenorm_quant: null pointer");
    FUSED_ROW_CHECKS("mmf_gatenorm_quant", D);
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(g, 16) && mmf_aligned(o, 16) && mmf_aligned(q, 16) && (ld_g * es) % 16 == 0 && (ld_o * es) % 16 == 0,
                MMF_ERR_ALIGN, "mmf_gatenorm_quant: rows must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    const size_t smem = (size_t)D * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        if (smem > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(gatenorm_quant_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        gatenorm_quant_kernel<T><<<(unsigned)M, FT, smem, (cudaStream_t)stream>>>((const T*)g, ld_g, (const T*)o, ld_o, gnorm_w, eps_g,
                                                                                    nw, eps_bl, q, dq, rowsum, (int)D);
    });
    MMF_LAUNCH_CHECK("gatenorm_quant_kernel");
    return MMF_OK;
}

extern "C" int mmf_swiglu_quant(const void* gate, const void* up, int64_t ld, int dtype, const float* nw, float eps_bl,
                                int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(gate && up && q && dq && rowsum, MMF_ERR_BAD_ARG, "mmf_swiglu_quant: null pointer");
    FUSED_ROW_CHECKS("mmf_swiglu_quant", D);
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(gate, 16) && mmf_aligned(up, 16) && mmf_aligned(q, 16) && (ld * es) % 16 == 0, MMF_ERR_ALIGN,
                "mmf_swiglu_quant: rows must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    const size_t smem = (size_t)D * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        if (smem > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(swiglu_quant_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        swiglu_quant_kernel<T><<<(unsigned)M, FT, smem, (cudaStream_t)stream>>>((const T*)gate, (const T*)up, ld, nw, eps_bl, q, dq,
                                                                                  rowsum, (int)D);
    });
    MMF_LAUNCH_CHECK("swiglu_quant_kernel");
    return MMF_OK;
}
