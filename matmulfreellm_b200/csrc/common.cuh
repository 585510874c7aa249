// Shared device/host helpers for libmmfree_b200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mmfree_b200.h"
#include <cuda/std/type_traits>

// ---------------------------------------------------------------------------------------
// host-side error plumbing
// ---------------------------------------------------------------------------------------
int mmf_set_error(int code, const char* fmt, ...);

#define MMF_REQUIRE(cond, code, ...)                       \
    do {                                                   \
        if (!(cond)) return mmf_set_error(code, __VA_ARGS__); \
    } while (0)

#define MMF_CUDA(...)                                                                   \
    do {                                                                                \
        cudaError_t e__ = (__VA_ARGS__);                                                \
        if (e__ != cudaSuccess) {                                                       \
            (void)cudaGetLastError(); /* do not leave the error for a later launch check */ \
            return mmf_set_error(MMF_ERR_CUDA, "%s failed: %s", #__VA_ARGS__, cudaGetErrorString(e__)); \
        }                                                                               \
    } while (0)

#define MMF_LAUNCH_CHECK(name)                                                          \
    do {                                                                                \
        cudaError_t e__ = cudaGetLastError();                                           \
        if (e__ != cudaSuccess)                                                         \
            return mmf_set_error(MMF_ERR_CUDA, "launch of %s failed: %s", name,         \
                                 cudaGetErrorString(e__));                              \
    } while (0)

static inline bool mmf_aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static inline bool mmf_dtype_ok(int dt) { return dt == MMF_F32 || dt == MMF_BF16 || dt == MMF_F16; }
static inline int mmf_dtype_size(int dt) { return dt == MMF_F32 ? 4 : 2; }

// Run `...` with `T` bound to the C++ type of dtype code `dt`.
#define MMF_DISPATCH(dt, T, ...)                         \
    switch (dt) {                                        \
        case MMF_F32: { using T = float; __VA_ARGS__; break; }          \
        case MMF_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
        default: { using T = __half; __VA_ARGS__; break; }              \
    }

// ---------------------------------------------------------------------------------------
// programmatic dependent launch: the kernels of a decode step are launched with the
// programmatic-stream-serialization attribute, so kernel N+1 may start (and run whatever does not
// depend on kernel N: barrier set-up, constants, the weight stream) while kernel N drains.  Every
// such kernel calls pdl_trigger() at its top and pdl_wait() before it touches memory written by
// its predecessors; pdl_wait() returns once those grids have completed and flushed.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t mmf_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---------------------------------------------------------------------------------------
// element conversion (round-to-nearest-even on store, exact on load)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// value of v after a round trip through T (models an intermediate tensor of dtype T)
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

// Two values rounded to T in place with one packed conversion; returns the two T values as 32 bits (a in the low
// half), which a caller that also stores them can write out without converting again.  No-op for T = float.
template <typename T> __device__ __forceinline__ uint32_t round_pair(float& a, float& b);
template <> __device__ __forceinline__ uint32_t round_pair<float>(float&, float&) { return 0u; }
template <> __device__ __forceinline__ uint32_t round_pair<__nv_bfloat16>(float& a, float& b) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&p);
    a = __uint_as_float(u << 16);
    b = __uint_as_float(u & 0xffff0000u);
    return u;
}
template <> __device__ __forceinline__ uint32_t round_pair<__half>(float& a, float& b) {
    const __half2 p = __floats2half2_rn(a, b);
    const float2 f = __half22float2(p);
    a = f.x;
    b = f.y;
    return *reinterpret_cast<const uint32_t*>(&p);
}
// V values (one 16-byte vector of T) rounded to T in place; `bits` receives the packed T values (16-bit T only)
template <typename T, int V>
__device__ __forceinline__ void round_vec(float (&x)[V], uint32_t (&bits)[V / 2]) {
#pragma unroll
    for (int i = 0; i < V; i += 2) bits[i / 2] = round_pair<T>(x[i], x[i + 1]);
}
// store a vector that round_vec has rounded: the packed bits for a 16-bit T, the values themselves for float
template <typename T, int V>
__device__ __forceinline__ void store_rounded(T* p, const float (&x)[V], const uint32_t (&bits)[V / 2]) {
    if constexpr (sizeof(T) == 2) *reinterpret_cast<uint4*>(p) = make_uint4(bits[0], bits[1], bits[2], bits[3]);
    else *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}

// ss += sum of x[i]^2 in fp64 for V values that round_vec has just rounded to T (`bits`: the packed T values).  For
// bf16 the fp64 operand is assembled from the 16 bits with two integer instructions per value — sign dropped (it is
// squared), exponent rebiased: ((b & 0x7fff) << 13) + (896 << 20) is the high word of the double, the low word is zero —
// instead of an fp32 -> fp64 conversion, which runs on the special-function pipe (16 results per clock and SM: the pipe
// that bounds the gate-norm and swiglu kernels on prompts).  A zero or subnormal bf16 value reads as about 2^-127, whose
// square, 1e-77, cannot reach the fp32 statistic.  The square and the sum are the same fp64 fused multiply-add as before.
template <typename T, int V>
__device__ __forceinline__ void sumsq_rounded(const float (&x)[V], const uint32_t (&bits)[V / 2], double& ss) {
    if constexpr (sizeof(T) == 2 && !cuda::std::is_same<T, __half>::value) {
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
            const uint32_t u = bits[i];
            const double d0 = __hiloint2double((int)(((u & 0x7fffu) << 13) + 0x38000000u), 0);
            const double d1 = __hiloint2double((int)(((u >> 3) & 0x0fffe000u) + 0x38000000u), 0);
            ss = fma(d0, d0, ss);
            ss = fma(d1, d1, ss);
        }
    } else {
#pragma unroll
        for (int i = 0; i < V; ++i) ss += (double)x[i] * (double)x[i];
    }
}

// int8 activation code clamp(rint(p), -128, 127) for |p| < 2^22 without conversion instructions: adding 1.5 * 2^23
// leaves the round-to-nearest-even integer in the low mantissa bits of the sum (same result as rintf + cast)
__device__ __forceinline__ int quant_code(float p) {
    const int iv = __float_as_int(__fadd_rn(p, 12582912.0f)) - 0x4B400000;
    return max(-128, min(127, iv));
}

// 16-byte vector of T: 4 floats or 8 halves
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); T v[N]; };

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&out)[16 / sizeof(T)]) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < (int)(16 / sizeof(T)); ++i) out[i] = to_f32(e[i]);
}

template <typename T>
__device__ __forceinline__ void store16(T* p, const float (&in)[16 / sizeof(T)]) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < (int)(16 / sizeof(T)); ++i) e[i] = from_f32<T>(in[i]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// ---------------------------------------------------------------------------------------
// block reductions (blockDim.x a multiple of 32, <= 1024); result broadcast to all threads
// `red` is shared scratch of >= 33 elements of T.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ double block_sum(double v, double* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // protect `red` from the previous use
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        double t = lane < nw ? red[lane] : 0.0;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        float t = lane < nw ? red[lane] : 0.0f;  // callers reduce non-negative values
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ int block_sum(int v, int* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    if (wid == 0) {
        int t = lane < nw ? red[lane] : 0;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ---------------------------------------------------------------------------------------
// the exact arithmetic of the quantisation path (mirrored by the CPU oracle): every step is
// a single IEEE round-to-nearest fp32 operation, never contracted into an fma.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float rstd_from_sumsq(double sumsq, int64_t K, float eps) {
    // K a power of two (2048, 4096 ...): scaling by 2^-n is the exact quotient, without the ~100-instruction fp64 division
    // that otherwise sits on the critical path of every row kernel of a decode step
    const double q = (K & (K - 1)) == 0 ? sumsq * __longlong_as_double((1023ll - (long long)(__ffsll((long long)K) - 1)) << 52)
                                        : sumsq / (double)K;
    const float mean = (float)q;
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
}
// e^-x and the reciprocal through the special-function unit (ex2.approx, rcp.approx: relative error about 2^-22 each).
// The results feed values that are rounded to the activation dtype right away, or compared at 1e-4, so the two extra
// units in the last place are invisible there, and each call is 6 instructions instead of more than 20.
__device__ __forceinline__ float exp_neg(float x) {
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(__fmul_rn(x, -1.4426950408889634f)));
    return p;
}
__device__ __forceinline__ float rcp_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float silu_mul(float x, float y) {
    // float(x) * float(y) / (1.0f + exp(-float(x)))
    return __fmul_rn(__fmul_rn(x, y), rcp_fast(__fadd_rn(1.0f, exp_neg(x))));
}
__device__ __forceinline__ float sigmoidf_(float x) { return rcp_fast(__fadd_rn(1.0f, exp_neg(x))); }
// the same on two values at once: the multiplies and adds are packed f32x2 instructions (each half is the scalar IEEE
// operation), the special-function calls stay per value.  No packed multiply here feeds an add directly (such a pair
// can be merged into a fused multiply-add, which rounds once instead of twice).
// One reciprocal serves both values: 1/a = b * (1/(ab)), 1/b = a * (1/(ab)) — three special-function instructions per
// pair instead of four (that pipe, at 16 results per clock and SM, is what bounds the gate-norm and swiglu kernels on
// prompts).  The exponents are limited to 2^60 so that the product stays finite (sigmoid(v) for v < -41.6 reads 2^-60
// instead of a smaller number).
__device__ __forceinline__ float2 sigmoid2(float2 x) {
    float2 t = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    t.x = fminf(t.x, 60.0f);
    t.y = fminf(t.y, 60.0f);
    float2 e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
    const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), e);
    const float r = rcp_fast(__fmul_rn(d.x, d.y));
    return __fmul2_rn(make_float2(d.y, d.x), make_float2(r, r));
}
__device__ __forceinline__ float2 silu_mul2(float2 x, float2 y) { return __fmul2_rn(__fmul2_rn(x, y), sigmoid2(x)); }

// ---------------------------------------------------------------------------------------
// HGRNBitAttention's gate math on a pair of channels (shared by the scan and the fused decode step, so that both
// produce the same bits):
//   f = round(sigmoid(f_raw)); with a lower bound lb: f = round(lb + round(round(1-lb)*f));
//   x = round(silu(i_raw) * round(1-f));            every round() is to the activation dtype TX
// ---------------------------------------------------------------------------------------
// a pair of 16-bit activations as one 32-bit register
template <typename T> struct Pair16 { using type = float2; };
template <> struct Pair16<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Pair16<__half> { using type = __half2; };
__device__ __forceinline__ float2 unpack2(__nv_bfloat162 v) {
    const uint32_t u = *reinterpret_cast<const uint32_t*>(&v);
    return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ float2 unpack2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ void pack2(__nv_bfloat162& d, float2 v) { d = __floats2bfloat162_rn(v.x, v.y); }
__device__ __forceinline__ void pack2(__half2& d, float2 v) { d = __floats2half2_rn(v.x, v.y); }

// sigmoid of four values with two reciprocals instead of four: 1/a = b * (1/(a*b)), 1/b = a * (1/(a*b)).  The caller
// keeps the arguments >= RAW_GATE_MIN so that the product a*b stays finite.
constexpr float RAW_GATE_MIN = -40.0f;
__device__ __forceinline__ void sigmoid_pairs(float2 g, float2 x, float2& sg, float2& sx) {
    const float2 nl2e = make_float2(-1.4426950408889634f, -1.4426950408889634f);
    const float2 tg = __fmul2_rn(g, nl2e), tx = __fmul2_rn(x, nl2e);
    float2 eg, ex;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(eg.x) : "f"(tg.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(eg.y) : "f"(tg.y));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex.x) : "f"(tx.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex.y) : "f"(tx.y));
    const float2 one = make_float2(1.0f, 1.0f);
    const float2 a = __fadd2_rn(one, eg), b = __fadd2_rn(one, ex);
    const float2 p = __fmul2_rn(a, b);
    const float2 r = make_float2(rcp_fast(p.x), rcp_fast(p.y));
    sg = __fmul2_rn(b, r);
    sx = __fmul2_rn(a, r);
}
// both raw projections of a channel pair limited to >= RAW_GATE_MIN (below it sigmoid and silu are zero to 17 digits),
// on the packed pair for a 16-bit dtype
__device__ __forceinline__ float2 raw_gate_floor(float2 v) { return make_float2(fmaxf(v.x, RAW_GATE_MIN), fmaxf(v.y, RAW_GATE_MIN)); }
__device__ __forceinline__ __nv_bfloat162 raw_gate_floor(__nv_bfloat162 v) { return __hmax2(v, __float2bfloat162_rn(RAW_GATE_MIN)); }
__device__ __forceinline__ __half2 raw_gate_floor(__half2 v) { return __hmax2(v, __float2half2_rn(RAW_GATE_MIN)); }

// In: xv = i_raw, f = f_raw of two adjacent channels, already passed through raw_gate_floor; out: xv = x_t, f = f_t.  With a 16-bit activation dtype the steps
// between two roundings run on the packed pair: the product, sum and difference of two 16-bit floats rounded once to
// 16 bits (mul / add / sub on the packed type) equal the fp32 operation followed by the rounding, because the fp32 result
// is exact or nowhere near a 16-bit rounding boundary.  lbv = lower bound, oml = round(1 - lb) (pass {0, 1} without one).
template <typename TX>
__device__ __forceinline__ void raw_gate_pair(float2& xv, float2& f, bool has_lb, float2 lbv, float2 oml) {
    float2 sg, sx;
    sigmoid_pairs(f, xv, sg, sx);
    float2 omf;
    if constexpr (sizeof(TX) == 2) {
        typename Pair16<TX>::type f16, lb16, oml16, one16, omf16, x16;
        pack2(f16, sg);
        if (has_lb) {
            pack2(lb16, lbv);                  // exact: both are values of TX already
            pack2(oml16, oml);
            f16 = __hadd2(lb16, __hmul2(oml16, f16));
        }
        pack2(one16, make_float2(1.0f, 1.0f));
        omf16 = __hsub2(one16, f16);
        f = unpack2(f16);
        omf = unpack2(omf16);
        pack2(x16, __fmul2_rn(__fmul2_rn(xv, omf), sx));
        xv = unpack2(x16);
    } else {
        f = sg;
        if (has_lb) {
            // scalar on purpose: a packed multiply feeding a packed add can be merged into a fused multiply-add
            f.x = __fadd_rn(lbv.x, __fmul_rn(oml.x, f.x));
            f.y = __fadd_rn(lbv.y, __fmul_rn(oml.y, f.y));
        }
        omf = make_float2(__fsub_rn(1.0f, f.x), __fsub_rn(1.0f, f.y));
        xv = __fmul2_rn(__fmul2_rn(xv, omf), sx);
    }
}
