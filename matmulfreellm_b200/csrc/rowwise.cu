// Row-wise kernels: BitLinear prologue (RMSNorm + int8 absmax quantisation), RMSNorm with
// residual, RMSNorm * swish-gate, SwiGLU, arg-max and embedding lookup.
//
// All of them are HBM-bound streaming kernels: one CTA per row, 16-byte vector loads, the
// row cached in shared memory as fp32 between the statistics pass and the output pass so
// that every input byte is read from HBM once.
#include "common.cuh"

namespace {

constexpr int ROW_THREADS = 256;

template <typename T, int V>
__device__ __forceinline__ void load_n(const T* p, float (&out)[V]) {
    if constexpr (V == 1) {
        out[0] = to_f32(*p);
    } else {
        static_assert(V == 16 / sizeof(T), "vector width");
        load16<T>(p, out);
    }
}
template <typename T, int V>
__device__ __forceinline__ void store_n(T* p, const float (&in)[V]) {
    if constexpr (V == 1) {
        *p = from_f32<T>(in[0]);
    } else {
        store16<T>(p, in);
    }
}

// -----------------------------------------------------------------------------------------
// RMSNorm + activation quantisation
// -----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(ROW_THREADS)
act_quant_kernel(const T* __restrict__ x, int64_t ld_x, const float* __restrict__ nw, int use_norm,
                 float eps, int8_t* __restrict__ q, float* __restrict__ dq,
                 int32_t* __restrict__ rowsum, int K) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    __shared__ float redf[33];
    __shared__ int redi[33];
    constexpr int V = 16 / sizeof(T);
    const int64_t m = blockIdx.x;
    const T* xr = x + m * ld_x;

    double ss = 0.0;
    for (int c = threadIdx.x * V; c < K; c += ROW_THREADS * V) {
        float v[V];
        load_n<T, V>(xr + c, v);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            row[c + i] = v[i];
            ss += (double)v[i] * (double)v[i];
        }
    }
    float rstd = 1.0f;
    if (use_norm) rstd = rstd_from_sumsq(block_sum(ss, redd), K, eps);

    float amax = 0.0f;
    for (int c = threadIdx.x * V; c < K; c += ROW_THREADS * V) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float y = row[c + i];
            if (use_norm) {
                y = __fmul_rn(y, rstd);
                if (nw) y = __fmul_rn(y, nw[c + i]);
            }
            row[c + i] = y;
            amax = fmaxf(amax, fabsf(y));
        }
    }
    amax = block_max(amax, redf);
    const float a = fmaxf(amax, 1e-5f);
    const float s = __fdiv_rn(127.0f, a);

    int lsum = 0;
    int8_t* qr = q + m * (int64_t)K;
    for (int c = threadIdx.x * V; c < K; c += ROW_THREADS * V) {
        int8_t codes[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int iv = quant_code(__fmul_rn(row[c + i], s));
            codes[i] = (int8_t)iv;
            lsum += iv;
        }
        if constexpr (V == 8) {
            *reinterpret_cast<uint2*>(qr + c) = *reinterpret_cast<const uint2*>(codes);
        } else {
            *reinterpret_cast<uint32_t*>(qr + c) = *reinterpret_cast<const uint32_t*>(codes);
        }
    }
    lsum = block_sum(lsum, redi);
    if (threadIdx.x == 0) {
        dq[m] = __fdiv_rn(a, 127.0f);
        rowsum[m] = lsum;
    }
}

// -----------------------------------------------------------------------------------------
// RMSNorm (+ residual, + residual_out)
// -----------------------------------------------------------------------------------------
template <typename T, typename R, int V>
__global__ void __launch_bounds__(ROW_THREADS)
rmsnorm_kernel(const T* __restrict__ x, const R* __restrict__ res, const float* __restrict__ w,
               float eps, T* __restrict__ y, R* __restrict__ res_out, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    const int64_t m = blockIdx.x;
    const T* xr = x + m * (int64_t)D;
    const R* rr = res ? res + m * (int64_t)D : nullptr;
    R* ro = res_out ? res_out + m * (int64_t)D : nullptr;
    constexpr int VR = (V == 1) ? 1 : 16 / sizeof(R);  // elements per 16-byte vector of R

    double ss = 0.0;
    for (int c = threadIdx.x * V; c < D; c += ROW_THREADS * V) {
        float v[V];
        load_n<T, V>(xr + c, v);
        if (rr) {
            // R vectors may be narrower than T vectors (fp32 residual with 16-bit x)
#pragma unroll
            for (int j = 0; j < V; j += VR) {
                float r[VR];
                load_n<R, VR>(rr + c + j, r);
#pragma unroll
                for (int i = 0; i < VR; ++i) v[j + i] = __fadd_rn(v[j + i], r[i]);
            }
        }
        if (ro) {
#pragma unroll
            for (int j = 0; j < V; j += VR) {
                float r[VR];
#pragma unroll
                for (int i = 0; i < VR; ++i) r[i] = v[j + i];
                store_n<R, VR>(ro + c + j, r);
            }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            row[c + i] = v[i];
            ss += (double)v[i] * (double)v[i];
        }
    }
    const float rstd = rstd_from_sumsq(block_sum(ss, redd), D, eps);
    T* yr = y + m * (int64_t)D;
    for (int c = threadIdx.x * V; c < D; c += ROW_THREADS * V) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float t = __fmul_rn(row[c + i], rstd);
            if (w) t = __fmul_rn(t, w[c + i]);
            o[i] = t;
        }
        store_n<T, V>(yr + c, o);
    }
}

// -----------------------------------------------------------------------------------------
// RMSNorm(x) * w * o * sigmoid(o)
// -----------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(ROW_THREADS)
swishgate_kernel(const T* __restrict__ x, const T* __restrict__ o, const float* __restrict__ w,
                 float eps, T* __restrict__ y, int D) {
    extern __shared__ __align__(16) float row[];
    __shared__ double redd[33];
    const int64_t m = blockIdx.x;
    const T* xr = x + m * (int64_t)D;
    const T* orow = o + m * (int64_t)D;
    double ss = 0.0;
    for (int c = threadIdx.x * V; c < D; c += ROW_THREADS * V) {
        float v[V];
        load_n<T, V>(xr + c, v);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            row[c + i] = v[i];
            ss += (double)v[i] * (double)v[i];
        }
    }
    const float rstd = rstd_from_sumsq(block_sum(ss, redd), D, eps);
    T* yr = y + m * (int64_t)D;
    for (int c = threadIdx.x * V; c < D; c += ROW_THREADS * V) {
        float g[V], out[V];
        load_n<T, V>(orow + c, g);
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float t = __fmul_rn(row[c + i], rstd);
            if (w) t = __fmul_rn(t, w[c + i]);
            t = __fmul_rn(t, g[i]);
            out[i] = __fmul_rn(t, sigmoidf_(g[i]));
        }
        store_n<T, V>(yr + c, out);
    }
}

// -----------------------------------------------------------------------------------------
// SwiGLU  out = x*y/(1+exp(-x))
// -----------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ x, int64_t ld_x, const T* __restrict__ y, int64_t ld_y,
              T* __restrict__ out, int64_t ld_out, int64_t M, int D) {
    const int per_row = D / V;
    const int64_t total = M * (int64_t)per_row;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / per_row;
        const int c = (int)(i - m * per_row) * V;
        float a[V], b[V], o[V];
        load_n<T, V>(x + m * ld_x + c, a);
        load_n<T, V>(y + m * ld_y + c, b);
#pragma unroll
        for (int k = 0; k < V; ++k) o[k] = silu_mul(a[k], b[k]);
        store_n<T, V>(out + m * ld_out + c, o);
    }
}

// -----------------------------------------------------------------------------------------
// arg-max per row (first index on ties) and embedding lookup
// -----------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
argmax_kernel(const T* __restrict__ logits, int64_t ld, int V, int64_t* __restrict__ idx, int vec16) {
    pdl_trigger();
    pdl_wait();
    __shared__ float sv[8];
    __shared__ int si[8];
    const T* r = logits + blockIdx.x * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    constexpr int VL = 16 / sizeof(T);
    if (vec16) {   // 16-byte loads; a thread's columns ascend, so '>' keeps the first maximum it meets
        for (int c = threadIdx.x * VL; c < V; c += blockDim.x * VL) {
            float v[VL];
            load16<T>(r + c, v);
#pragma unroll
            for (int i = 0; i < VL; ++i)
                if (c + i < V && (v[i] > best || (v[i] == best && c + i < bi))) { best = v[i]; bi = c + i; }
        }
    } else {
        for (int c = threadIdx.x; c < V; c += blockDim.x) {
            const float v = to_f32(r[c]);
            if (v > best || (v == best && c < bi)) { best = v; bi = c; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int wdx = 1; wdx < 8; ++wdx)
            if (sv[wdx] > best || (sv[wdx] == best && si[wdx] < bi)) { best = sv[wdx]; bi = si[wdx]; }
        idx[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// Nucleus (top-p) sampling of one token per row, deterministic given one uniform number per row:
//   p_i = softmax(logits_i / temperature); keep the smallest set of most probable tokens whose mass reaches top_p
//   (all tokens with p_i >= tau, tau found by bisection on the float bit pattern; tokens tied at tau are all kept);
//   the sample is the first kept token, in index order, at which the running kept mass exceeds u * (kept mass).
// Sums are accumulated in fp64 in a fixed order, so the result does not depend on scheduling.
template <typename T>
__global__ void __launch_bounds__(256)
sample_top_p_kernel(const T* __restrict__ logits, int64_t ld, int V, float inv_temp, float top_p,
                    const float* __restrict__ uniforms, int64_t* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    __shared__ double red[40];
    __shared__ float redf[40];
    __shared__ double s_part[256];
    __shared__ int s_found;
    const T* r = logits + blockIdx.x * ld;
    const int chunk = (V + 255) / 256;
    const int c0 = min(V, (int)threadIdx.x * chunk), c1 = min(V, c0 + chunk);   // this thread's contiguous tokens
    float mx = -INFINITY;
    for (int c = c0; c < c1; ++c) mx = fmaxf(mx, __fmul_rn(to_f32(r[c]), inv_temp));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) redf[threadIdx.x >> 5] = mx;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) mx = fmaxf(mx, redf[w]);
    auto prob = [&](int c) { return expf(__fsub_rn(__fmul_rn(to_f32(r[c]), inv_temp), mx)); };
    auto mass_ge = [&](float tau) {          // total probability (unnormalised) of the tokens with p >= tau
        double acc = 0.0;
        for (int c = c0; c < c1; ++c) {
            const float p = prob(c);
            if (p >= tau) acc += (double)p;
        }
        return block_sum(acc, red);
    };
    const double total = mass_ge(0.0f);
    const double want = (double)top_p * total;
    uint32_t lo = 0u, hi = __float_as_uint(1.0f) + 1u;    // mass_ge(lo) >= want > mass_ge(hi)  (p <= 1 everywhere)
    while (hi - lo > 1u) {
        const uint32_t mid = lo + (hi - lo) / 2u;
        if (mass_ge(__uint_as_float(mid)) >= want) lo = mid; else hi = mid;
    }
    const float tau = __uint_as_float(lo);
    // kept mass per thread, then an exclusive prefix in thread order (= token order)
    double part = 0.0;
    for (int c = c0; c < c1; ++c) {
        const float p = prob(c);
        if (p >= tau) part += (double)p;
    }
    s_part[threadIdx.x] = part;
    if (threadIdx.x == 0) s_found = 0x7fffffff;
    __syncthreads();
    double before = 0.0, kept = 0.0;
    for (int t = 0; t < 256; ++t) {
        if (t == (int)threadIdx.x) before = kept;
        kept += s_part[t];
    }
    const double target = (double)uniforms[blockIdx.x] * kept;
    if (part > 0.0 && target >= before && target < before + part) {
        double run = before;
        for (int c = c0; c < c1; ++c) {
            const float p = prob(c);
            if (p >= tau) {
                run += (double)p;
                if (run > target) { atomicMin(&s_found, c); break; }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // rounding may leave the last interval open at its end: fall back to the last kept token
        int found = s_found;
        if (found == 0x7fffffff) {
            for (int c = V - 1; c >= 0; --c)
                if (prob(c) >= tau) { found = c; break; }
        }
        out[blockIdx.x] = found == 0x7fffffff ? 0 : found;
    }
}

__global__ void __launch_bounds__(128)
embedding_kernel(const uint8_t* __restrict__ table, int64_t V, int64_t row_bytes,
                 const int64_t* __restrict__ ids, uint8_t* __restrict__ out, int vec16) {
    pdl_trigger();
    pdl_wait();
    int64_t id = ids[blockIdx.x];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);  // clamp instead of faulting on a bad id
    const uint8_t* src = table + id * row_bytes;
    uint8_t* dst = out + blockIdx.x * row_bytes;
    if (vec16) {
        for (int64_t b = threadIdx.x * 16; b < row_bytes; b += blockDim.x * 16)
            *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(src + b);
    } else {
        for (int64_t b = threadIdx.x; b < row_bytes; b += blockDim.x) dst[b] = src[b];
    }
}

}  // namespace

// =========================================================================================
// C ABI
// =========================================================================================
extern "C" int mmf_act_quant(const void* x, int dtype, int64_t ld_x, const float* norm_w,
                             int use_norm, float eps, int8_t* q, float* dq, int32_t* rowsum,
                             int64_t M, int64_t K, void* stream) {
    MMF_REQUIRE(x && q && dq && rowsum, MMF_ERR_BAD_ARG, "mmf_act_quant: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_act_quant: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && K > 0 && K <= 16384 && K % 16 == 0, MMF_ERR_BAD_SHAPE,
                "mmf_act_quant: need 0 < K <= 16384, K %% 16 == 0 (K=%lld, M=%lld)", (long long)K,
                (long long)M);
    MMF_REQUIRE(ld_x >= K, MMF_ERR_BAD_SHAPE, "mmf_act_quant: ld_x < K");
    MMF_REQUIRE(mmf_aligned(x, 16) && (ld_x * mmf_dtype_size(dtype)) % 16 == 0 && mmf_aligned(q, 16),
                MMF_ERR_ALIGN, "mmf_act_quant: x rows and q must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)K * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        if (smem > 48 * 1024)
            MMF_CUDA(cudaFuncSetAttribute(act_quant_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MMF_CUDA(mmf_launch_pdl(act_quant_kernel<T>, dim3((unsigned)M), dim3(ROW_THREADS), smem, st, (const T*)x, ld_x, norm_w, use_norm, eps, q,
                                                                     dq, rowsum, (int)K));
    });
    MMF_LAUNCH_CHECK("act_quant_kernel");
    return MMF_OK;
}

template <typename T, typename R>
static int launch_rmsnorm(const void* x, const void* res, const float* w, float eps, void* y, void* res_out,
                          int64_t M, int64_t D, cudaStream_t st) {
    const size_t smem = (size_t)D * sizeof(float);
    constexpr int VT = 16 / sizeof(T);
    const bool vec = D % VT == 0 && mmf_aligned(x, 16) && mmf_aligned(y, 16) && (!res || mmf_aligned(res, 16)) &&
                     (!res_out || mmf_aligned(res_out, 16));
    if (vec) {
        if (smem > 48 * 1024)
            MMF_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<T, R, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        rmsnorm_kernel<T, R, VT><<<(unsigned)M, ROW_THREADS, smem, st>>>((const T*)x, (const R*)res, w, eps, (T*)y,
                                                                         (R*)res_out, (int)D);
    } else {
        if (smem > 48 * 1024)
            MMF_CUDA(cudaFuncSetAttribute(rmsnorm_kernel<T, R, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        rmsnorm_kernel<T, R, 1><<<(unsigned)M, ROW_THREADS, smem, st>>>((const T*)x, (const R*)res, w, eps, (T*)y,
                                                                        (R*)res_out, (int)D);
    }
    MMF_LAUNCH_CHECK("rmsnorm_kernel");
    return MMF_OK;
}

extern "C" int mmf_rmsnorm(const void* x, int dtype, const void* residual, int res_dtype, const float* w,
                           float eps, void* y, void* residual_out, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(x && y, MMF_ERR_BAD_ARG, "mmf_rmsnorm: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_rmsnorm: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && D > 0 && D <= 32768, MMF_ERR_BAD_SHAPE, "mmf_rmsnorm: need 0 < D <= 32768");
    const bool has_res = residual || residual_out;
    if (has_res)
        MMF_REQUIRE(res_dtype == dtype || res_dtype == MMF_F32, MMF_ERR_BAD_ARG,
                    "mmf_rmsnorm: residual dtype must equal x dtype or be fp32");
    if (M == 0) return MMF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool res_f32 = has_res && res_dtype == MMF_F32;
    int rc = MMF_OK;
    MMF_DISPATCH(dtype, T, {
        if (res_f32)
            rc = launch_rmsnorm<T, float>(x, residual, w, eps, y, residual_out, M, D, st);
        else
            rc = launch_rmsnorm<T, T>(x, residual, w, eps, y, residual_out, M, D, st);
    });
    return rc;
}

extern "C" int mmf_rmsnorm_swishgate(const void* x, const void* o, int dtype, const float* w, float eps, void* y,
                                     int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(x && o && y, MMF_ERR_BAD_ARG, "mmf_rmsnorm_swishgate: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_rmsnorm_swishgate: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && D > 0 && D <= 32768, MMF_ERR_BAD_SHAPE, "mmf_rmsnorm_swishgate: need 0 < D <= 32768");
    if (M == 0) return MMF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)D * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        constexpr int VT = 16 / sizeof(T);
        const bool vec = D % VT == 0 && mmf_aligned(x, 16) && mmf_aligned(o, 16) && mmf_aligned(y, 16);
        if (vec) {
            if (smem > 48 * 1024)
                MMF_CUDA(cudaFuncSetAttribute(swishgate_kernel<T, VT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            swishgate_kernel<T, VT><<<(unsigned)M, ROW_THREADS, smem, st>>>((const T*)x, (const T*)o, w, eps, (T*)y, (int)D);
        } else {
            if (smem > 48 * 1024)
                MMF_CUDA(cudaFuncSetAttribute(swishgate_kernel<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            swishgate_kernel<T, 1><<<(unsigned)M, ROW_THREADS, smem, st>>>((const T*)x, (const T*)o, w, eps, (T*)y, (int)D);
        }
    });
    MMF_LAUNCH_CHECK("swishgate_kernel");
    return MMF_OK;
}

extern "C" int mmf_swiglu(const void* x, int64_t ld_x, const void* y, int64_t ld_y, void* out, int64_t ld_out,
                          int dtype, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(x && y && out, MMF_ERR_BAD_ARG, "mmf_swiglu: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_swiglu: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && D > 0 && D < (1ll << 31) && ld_x >= D && ld_y >= D && ld_out >= D, MMF_ERR_BAD_SHAPE,
                "mmf_swiglu: bad sizes");
    if (M == 0) return MMF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int es = mmf_dtype_size(dtype);
    MMF_DISPATCH(dtype, T, {
        constexpr int VT = 16 / sizeof(T);
        const bool vec = D % VT == 0 && mmf_aligned(x, 16) && mmf_aligned(y, 16) && mmf_aligned(out, 16) &&
                         (ld_x * es) % 16 == 0 && (ld_y * es) % 16 == 0 && (ld_out * es) % 16 == 0;
        const int64_t work = M * (D / (vec ? VT : 1));
        const unsigned grid = (unsigned)((work + 255) / 256 < 148 * 16 ? (work + 255) / 256 : 148 * 16);
        if (vec)
            swiglu_kernel<T, VT><<<grid, 256, 0, st>>>((const T*)x, ld_x, (const T*)y, ld_y, (T*)out, ld_out, M, (int)D);
        else
            swiglu_kernel<T, 1><<<grid, 256, 0, st>>>((const T*)x, ld_x, (const T*)y, ld_y, (T*)out, ld_out, M, (int)D);
    });
    MMF_LAUNCH_CHECK("swiglu_kernel");
    return MMF_OK;
}

extern "C" int mmf_argmax_rows(const void* logits, int dtype, int64_t ld, int64_t M, int64_t V, int64_t* idx,
                               void* stream) {
    MMF_REQUIRE(logits && idx, MMF_ERR_BAD_ARG, "mmf_argmax_rows: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_argmax_rows: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && V > 0 && V < (1ll << 31) && ld >= V, MMF_ERR_BAD_SHAPE, "mmf_argmax_rows: bad sizes");
    if (M == 0) return MMF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int es = mmf_dtype_size(dtype);
    const int vec16 = mmf_aligned(logits, 16) && (ld * es) % 16 == 0 && V % (16 / es) == 0;
    MMF_DISPATCH(dtype, T, { MMF_CUDA(mmf_launch_pdl(argmax_kernel<T>, dim3((unsigned)M), dim3(256), 0, st, (const T*)logits, ld, (int)V, idx, vec16)); });
    MMF_LAUNCH_CHECK("argmax_kernel");
    return MMF_OK;
}

extern "C" int mmf_embedding(const void* table, int dtype, int64_t V, int64_t D, const int64_t* ids, void* out,
                             int64_t M, void* stream) {
    MMF_REQUIRE(table && ids && out, MMF_ERR_BAD_ARG, "mmf_embedding: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_embedding: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && V > 0 && D > 0, MMF_ERR_BAD_SHAPE, "mmf_embedding: bad sizes");
    if (M == 0) return MMF_OK;
    const int64_t row_bytes = D * mmf_dtype_size(dtype);
    const int vec16 = row_bytes % 16 == 0 && mmf_aligned(table, 16) && mmf_aligned(out, 16);
    MMF_CUDA(mmf_launch_pdl(embedding_kernel, dim3((unsigned)M), dim3(128), 0, (cudaStream_t)stream, (const uint8_t*)table, V, row_bytes, ids,
                                                                    (uint8_t*)out, vec16));
    MMF_LAUNCH_CHECK("embedding_kernel");
    return MMF_OK;
}

extern "C" int mmf_sample_top_p(const void* logits, int dtype, int64_t ld, float temperature, float top_p, const float* uniforms,
                                int64_t* idx, int64_t M, int64_t V, void* stream) {
    MMF_REQUIRE(logits && uniforms && idx, MMF_ERR_BAD_ARG, "mmf_sample_top_p: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_sample_top_p: unknown dtype %d", dtype);
    MMF_REQUIRE(M >= 0 && V > 0 && V < (1ll << 31) && ld >= V, MMF_ERR_BAD_SHAPE, "mmf_sample_top_p: bad sizes");
    MMF_REQUIRE(temperature > 0.0f && top_p >= 0.0f, MMF_ERR_BAD_ARG, "mmf_sample_top_p: need temperature > 0 and top_p >= 0");
    if (M == 0) return MMF_OK;
    const float inv_temp = 1.0f / temperature;
    MMF_DISPATCH(dtype, T, {
        MMF_CUDA(mmf_launch_pdl(sample_top_p_kernel<T>, dim3((unsigned)M), dim3(256), 0, (cudaStream_t)stream, (const T*)logits, ld, (int)V,
                                inv_temp, top_p < 1.0f ? top_p : 1.0f, uniforms, idx));
    });
    MMF_LAUNCH_CHECK("sample_top_p_kernel");
    return MMF_OK;
}
