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
//   decode_mix    : single-token step of the token mixer: gate math, state update in place, then
//                   gatenorm_quant — one kernel between the i/f/g contraction and o_proj
// (for T > 1 the gate math of the recurrence is fused into the scan kernel, hgrn.cu)
//
// These kernels are latency chains (one CTA per token row, a handful of block-wide reductions), so
// the row lives in registers (<= 32 values per thread), the constant norm weights are copied to
// shared memory BEFORE the grid-dependency wait (they do not depend on the preceding kernel), and
// every block reduction costs a single __syncthreads.
#include "common.cuh"

namespace {

constexpr int FT = 256;        // threads per row CTA
constexpr int FW = FT / 32;    // warps
constexpr int MAX_PER = 32;    // most row values a thread can hold -> D <= FT * MAX_PER = 8192
constexpr int MAX_D = FT * MAX_PER;
// Kernels are compiled for P = 8, 16, 24 and 32 row values per thread (D <= 2048, 4096, 6144, 8192): the row lives in
// registers, so the smaller instantiations leave room for more resident CTAs.

// A row is worked on by RT threads (RT / 32 warps): the whole CTA (RT = FT: one row at a time, decode steps, long
// rows) or a quarter of it (RT = 64: four rows side by side — a thread then holds four times as many values of its
// row, and the per-row cost of the reductions below, a good part of all instructions at 8 values per thread, is spread
// over four times as many).  The threads of a row meet at a barrier of their own.
template <int RT> __device__ __forceinline__ void row_sync() {
    if constexpr (RT == FT) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + (int)(threadIdx.x / RT)), "n"(RT) : "memory");
}
// One-sync row reductions: warp shuffle, lane 0 parks the partial in a slot that is used once per row,
// one barrier, then every thread folds the RT / 32 partials in a fixed order.
template <int K, int RT>
__device__ __forceinline__ void block_sum_d(double (&v)[K], double* slot /* K*FW, 16-byte aligned */) {
    constexpr int RW = RT / 32;
    const int lane = threadIdx.x & 31, wid = (threadIdx.x % RT) >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) slot[k * RW + wid] = v[k];
    }
    row_sync<RT>();
#pragma unroll
    for (int k = 0; k < K; ++k) {
        double t = 0.0;
#pragma unroll
        for (int w = 0; w < RW; w += 2) {
            const double2 p = *reinterpret_cast<const double2*>(slot + k * RW + w);
            t += p.x;
            t += p.y;
        }
        v[k] = t;
    }
}
// maximum of non-negative, non-NaN floats: their bit patterns order like unsigned integers, so one warp-wide
// integer reduction instruction replaces five shuffle + max rounds
template <int K, int RT>
__device__ __forceinline__ void block_max_f(float (&v)[K], float* slot) {
    constexpr int RW = RT / 32;
    const int lane = threadIdx.x & 31, wid = (threadIdx.x % RT) >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v[k])));
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) slot[k * RW + wid] = v[k];
    }
    row_sync<RT>();
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = 0.0f;
        if constexpr (RW >= 4) {
#pragma unroll
            for (int w = 0; w < RW; w += 4) {
                const float4 p = *reinterpret_cast<const float4*>(slot + k * RW + w);
                t = fmaxf(fmaxf(t, p.x), fmaxf(p.y, fmaxf(p.z, p.w)));
            }
        } else {
            const float2 p = *reinterpret_cast<const float2*>(slot + k * RW);
            t = fmaxf(p.x, p.y);
        }
        v[k] = t;
    }
}
// row-wide integer sums; only the row's first thread receives them (it is the one that writes them out)
template <int K, int RT>
__device__ __forceinline__ void block_sum_i_t0(int (&v)[K], int* slot) {
    constexpr int RW = RT / 32;
    const int lane = threadIdx.x & 31, wid = (threadIdx.x % RT) >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = __reduce_add_sync(0xffffffffu, v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) slot[k * RW + wid] = v[k];
    }
    row_sync<RT>();
    if (threadIdx.x % RT == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            int t = 0;
            if constexpr (RW >= 4) {
#pragma unroll
                for (int w = 0; w < RW; w += 4) {
                    const int4 p = *reinterpret_cast<const int4*>(slot + k * RW + w);
                    t += (p.x + p.y) + (p.z + p.w);
                }
            } else {
                const int2 p = *reinterpret_cast<const int2*>(slot + k * RW);
                t = p.x + p.y;
            }
            v[k] = t;
        }
    }
}

struct __align__(16) RedScratch {       // each member is written once per row and at least two barriers lie between two uses -> no extra barrier
    double d0[3 * FW], d1[3 * FW];
    float f0[3 * FW];
    int i0[3 * FW];
};

// copy `n` floats (or ones, if src is null) into shared memory; all threads take part
__device__ __forceinline__ void stage_weights(float* dst, const float* src, int n) {
    for (int i = threadIdx.x * 4; i < n; i += FT * 4) {
        float4 v = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (src) v = *reinterpret_cast<const float4*>(src + i);
        *reinterpret_cast<float4*>(dst + i) = v;
    }
}

// V consecutive staged weights (16-byte aligned: columns start at multiples of V, D is a multiple of 16) as vector loads
template <int V>
__device__ __forceinline__ void lds_weights(const float* p, float (&w)[V]) {
#pragma unroll
    for (int i = 0; i < V; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(p + i);
        w[i] = t.x; w[i + 1] = t.y; w[i + 2] = t.z; w[i + 3] = t.w;
    }
}

// asynchronous 16-byte copy global -> shared memory (no register staging) and its group bookkeeping
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// iterate over the 16-byte vectors of a row held as v[P] (P: the enclosing template parameter): vector `it` of this thread starts at column c
// (RT, the threads per row, is a template parameter or constant of the enclosing function)
#define ROW_FOREACH(V, D, it, c) \
    _Pragma("unroll") for (int it = 0, c = (int)(threadIdx.x % RT) * (V); it < P / (V); ++it, c += RT * (V)) if (c < (D))

// BitLinear prologue on a register-resident row `v` (values already in T precision): shared sum of squares
// `ss`, then per projection g: y = (v*rstd)*nw_g, absmax -> scale -> int8 codes, dq, rowsum.
template <int V, int G, int P, int RT = FT>
__device__ __forceinline__ void bitlinear_prologue(float (&v)[P], int D, double ss, float eps, const float* snw /* smem [G][D] */,
                                                   int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t m, RedScratch& red) {
    double s1[1] = {ss};
    block_sum_d<1, RT>(s1, red.d1);
    const float rstd = rstd_from_sumsq(s1[0], D, eps);
    float amax[G];
#pragma unroll
    for (int g = 0; g < G; ++g) amax[g] = 0.0f;
    // independent fp32 multiplies below are issued two at a time (packed f32x2 instructions: each half is the same
    // IEEE round-to-nearest operation as the scalar instruction); a multiply whose result feeds an add is never packed
    const float2 rstd2 = make_float2(rstd, rstd);
    ROW_FOREACH(V, D, it, c) {
#pragma unroll
        for (int i = 0; i < V; i += 2) {   // the row is kept normalised from here on
            const float2 t = __fmul2_rn(make_float2(v[it * V + i], v[it * V + i + 1]), rstd2);
            v[it * V + i] = t.x;
            v[it * V + i + 1] = t.y;
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float w[V];
            lds_weights<V>(snw + g * D + c, w);
#pragma unroll
            for (int i = 0; i < V; i += 2) {
                const float2 y = __fmul2_rn(make_float2(v[it * V + i], v[it * V + i + 1]), make_float2(w[i], w[i + 1]));
                if constexpr (G == 1) {   // a single projection: keep y itself for the second pass
                    v[it * V + i] = y.x;
                    v[it * V + i + 1] = y.y;
                }
                amax[g] = fmaxf(amax[g], fmaxf(fabsf(y.x), fabsf(y.y)));
            }
        }
    }
    block_max_f<G, RT>(amax, red.f0);
    int lsum[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const float a = fmaxf(amax[g], 1e-5f);
        const float s = __fdiv_rn(127.0f, a);
        int8_t* qr = q + ((int64_t)g * M + m) * D;
        lsum[g] = 0;
        ROW_FOREACH(V, D, it, c) {
            uint32_t words[V / 4];
            float w[V];
            if constexpr (G > 1) lds_weights<V>(snw + g * D + c, w);
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                int iv[4];
#pragma unroll
                for (int j = 0; j < 4; j += 2) {
                    float2 y = make_float2(v[it * V + i + j], v[it * V + i + j + 1]);
                    if constexpr (G > 1) y = __fmul2_rn(y, make_float2(w[i + j], w[i + j + 1]));
                    // |y * s| <= 127 * (1 + 2^-23) because a >= |y|: the rounded code needs no clamp.  Adding 1.5 * 2^23
                    // leaves the code, rounded to nearest even, in the low byte of the sum.  These two steps stay scalar:
                    // a packed multiply followed by a packed add can be merged into one fused multiply-add, which would
                    // round the exact product instead of the rounded one.
                    iv[j] = __float_as_int(__fadd_rn(__fmul_rn(y.x, s), 12582912.0f));
                    iv[j + 1] = __float_as_int(__fadd_rn(__fmul_rn(y.y, s), 12582912.0f));
                }
                // low bytes of the four codes -> one word; its signed byte sum joins the row's code sum in one instruction
                const uint32_t word = __byte_perm(__byte_perm(iv[0], iv[1], 0x0040), __byte_perm(iv[2], iv[3], 0x0040), 0x5410);
                words[i / 4] = word;
                lsum[g] = __dp4a((int)word, 0x01010101, lsum[g]);
            }
            if constexpr (V == 8) *reinterpret_cast<uint2*>(qr + c) = make_uint2(words[0], words[1]);
            else *reinterpret_cast<uint32_t*>(qr + c) = words[0];
        }
        if (threadIdx.x % RT == 0) dq[(int64_t)g * M + m] = __fdiv_rn(a, 127.0f);
    }
    block_sum_i_t0<G, RT>(lsum, red.i0);
    if (threadIdx.x % RT == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) rowsum[(int64_t)g * M + m] = lsum[g];
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
    int gsplit;                            // 1: grid.y = G CTAs per row, CTA y does projection y alone (decode-sized calls: the G
                                           //    prologues of a row run side by side instead of one after the other)
#ifdef MMF_EXPERIMENTS
    long long* trace;                      // experiments build: 8 global-timer stamps of CTA 0 per launch (see mmf_row_trace)
#endif
};

#ifdef MMF_EXPERIMENTS
__device__ __forceinline__ long long row_now() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define ROW_TRACE(slot) do { if (trace) trace[slot] = row_now(); } while (0)
#else
#define ROW_TRACE(slot) do { } while (0)
#endif

template <typename T, int P, int LAT, int RT = FT>
__global__ void __launch_bounds__(FT, LAT)
prenorm_quant_kernel(PrenormArgs a) {
    extern __shared__ __align__(16) float sw[];   // [1 + G][D]: block norm weight, then the BitLinear norm weights
    constexpr int RPC = FT / RT;                  // rows this CTA works on side by side
    __shared__ RedScratch reds[RPC];
    RedScratch& red = reds[threadIdx.x / RT];
    const int rg = threadIdx.x / RT;
    constexpr int V = 16 / sizeof(T);
    const int D = a.D;
#ifdef MMF_EXPERIMENTS
    long long* trace = nullptr;
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && a.trace) {
        const int idx = atomicAdd(reinterpret_cast<int*>(a.trace), 1);
        if (idx < 1000) trace = a.trace + 8 + 8 * idx;
    }
#endif
    ROW_TRACE(0);
    pdl_trigger();
    const int gy = a.gsplit ? blockIdx.y : 0;          // projection of this CTA when the projections are split over CTAs
    const int Gs = a.gsplit ? 1 : a.G;                 // projections this CTA quantises
    stage_weights(sw, a.norm_w, D);
    for (int g = 0; g < Gs; ++g) stage_weights(sw + (1 + g) * D, a.nws[gy + g], D);
    ROW_TRACE(1);
    pdl_wait();
    ROW_TRACE(2);
    __syncthreads();

    // Row loop (LAT = 0): the CTA's next row travels global -> shared memory by cp.async while the current one is
    // processed (thread-private 16-byte slots: no barrier, only the thread's own wait)
    T* sx = reinterpret_cast<T*>(sw + (1 + Gs) * D) + (size_t)rg * 2 * D;   // per row in flight: [D] x row, [D] residual row (LAT = 0 only)
    T* sr = sx + D;
    auto fetch = [&](int64_t row) {
        ROW_FOREACH(V, D, it, c) {
            cp_async16(sx + c, reinterpret_cast<const T*>(a.x) + row * a.ld_x + c);
            if (a.res) cp_async16(sr + c, reinterpret_cast<const T*>(a.res) + row * a.ld_res + c);
        }
        cp_async_commit();
    };
    const int64_t row0 = (int64_t)blockIdx.x * RPC + rg, row_step = (int64_t)gridDim.x * RPC;
    if (LAT == 0 && row0 < a.M) fetch(row0);
    // a CTA takes rows blockIdx.x (* RPC + its row slot), + gridDim.x (* RPC), ...: with many rows the staged norm weights are reused
    for (int64_t m = row0; m < a.M; m += row_step) {
        const T* xr = LAT == 0 ? sx : reinterpret_cast<const T*>(a.x) + m * a.ld_x;
        const T* rr = a.res ? (LAT == 0 ? sr : reinterpret_cast<const T*>(a.res) + m * a.ld_res) : nullptr;
        if (LAT == 0) cp_async_wait_all();
        T* ro = (a.res_out && gy == 0) ? reinterpret_cast<T*>(a.res_out) + m * (int64_t)D : nullptr;
        float v[P];
        double ss[1] = {0.0};
        ROW_FOREACH(V, D, it, c) {
            float x[V];
            load16<T>(xr + c, x);
            if (rr) {
                float r[V];
                load16<T>(rr + c, r);
    #pragma unroll
                for (int i = 0; i < V; i += 2) {
                    const float2 t = __fadd2_rn(make_float2(x[i], x[i + 1]), make_float2(r[i], r[i + 1]));
                    x[i] = t.x;
                    x[i + 1] = t.y;
                }
            }
            if (ro || a.round_sum_first) {
                float xr_[V];
                uint32_t bits[V / 2];
    #pragma unroll
                for (int i = 0; i < V; ++i) xr_[i] = x[i];
                round_vec<T, V>(xr_, bits);
                if (ro) store_rounded<T, V>(ro + c, xr_, bits);
                if (a.round_sum_first) {
    #pragma unroll
                    for (int i = 0; i < V; ++i) x[i] = xr_[i];
                }
            }
    #pragma unroll
            for (int i = 0; i < V; ++i) {
                v[it * V + i] = x[i];
                ss[0] += (double)x[i] * (double)x[i];
            }
        }
        if (LAT == 0 && m + row_step < a.M) fetch(m + row_step);   // this thread's slots have just been read
        ROW_TRACE(3);
        block_sum_d<1, RT>(ss, red.d0);
        ROW_TRACE(4);
        const float rstd1 = rstd_from_sumsq(ss[0], D, a.eps_norm);
        T* yo = (a.y_out && gy == 0) ? reinterpret_cast<T*>(a.y_out) + m * (int64_t)D : nullptr;
        double ss2 = 0.0;
        ROW_FOREACH(V, D, it, c) {
            float o[V], w[V];
            uint32_t bits[V / 2];
            lds_weights<V>(sw + c, w);
#pragma unroll
            for (int i = 0; i < V; i += 2) {
                const float2 t = __fmul2_rn(__fmul2_rn(make_float2(v[it * V + i], v[it * V + i + 1]), make_float2(rstd1, rstd1)),
                                            make_float2(w[i], w[i + 1]));
                o[i] = t.x;
                o[i + 1] = t.y;
            }
            round_vec<T, V>(o, bits);
#pragma unroll
            for (int i = 0; i < V; ++i) v[it * V + i] = o[i];
            sumsq_rounded<T, V>(o, bits, ss2);
            if (yo) store_rounded<T, V>(yo + c, o, bits);
        }
        ROW_TRACE(5);
        if (a.gsplit)
            bitlinear_prologue<V, 1, P, RT>(v, D, ss2, a.eps_bl, sw + D, a.q + (int64_t)gy * a.M * D, a.dq + (int64_t)gy * a.M,
                                            a.rowsum + (int64_t)gy * a.M, a.M, m, red);
        else if (a.G == 3) bitlinear_prologue<V, 3, P, RT>(v, D, ss2, a.eps_bl, sw + D, a.q, a.dq, a.rowsum, a.M, m, red);
        else if (a.G == 1) bitlinear_prologue<V, 1, P, RT>(v, D, ss2, a.eps_bl, sw + D, a.q, a.dq, a.rowsum, a.M, m, red);
        ROW_TRACE(6);
    }
    ROW_TRACE(7);
}

// y = round_T( ((g*rstd)*w) * o * sigmoid(o) ), then BitLinear prologue.  `ov` holds the gate row o in registers.
template <typename T, int V, int P, int RT = FT>
__device__ __forceinline__ void gatenorm_tail(float (&gv)[P], const float (&ov)[P], double ssg, int D, float eps_g, float eps_bl,
                                              const float* sw /* [2][D]: g_norm weight, BitLinear norm weight */, int8_t* q, float* dq,
                                              int32_t* rowsum, int64_t M, int64_t m, RedScratch& red) {
    double s0[1] = {ssg};
    block_sum_d<1, RT>(s0, red.d0);
    const float rstd = rstd_from_sumsq(s0[0], D, eps_g);
    double ss2 = 0.0;
    ROW_FOREACH(V, D, it, c) {
        float w[V], t[V];
        uint32_t bits[V / 2];
        lds_weights<V>(sw + c, w);
#pragma unroll
        for (int i = 0; i < V; i += 2) {
            const float2 o = make_float2(ov[it * V + i], ov[it * V + i + 1]);
            float2 y = __fmul2_rn(__fmul2_rn(make_float2(gv[it * V + i], gv[it * V + i + 1]), make_float2(rstd, rstd)),
                                  make_float2(w[i], w[i + 1]));
            y = __fmul2_rn(__fmul2_rn(y, o), sigmoid2(o));
            t[i] = y.x;
            t[i + 1] = y.y;
        }
        round_vec<T, V>(t, bits);
#pragma unroll
        for (int i = 0; i < V; ++i) gv[it * V + i] = t[i];
        sumsq_rounded<T, V>(t, bits, ss2);
    }
    bitlinear_prologue<V, 1, P, RT>(gv, D, ss2, eps_bl, sw + D, q, dq, rowsum, M, m, red);
}

template <typename T, int P, int LAT, int RT = FT>
__global__ void __launch_bounds__(FT, LAT)
gatenorm_quant_kernel(const T* __restrict__ gx, int64_t ld_g, const T* __restrict__ o, int64_t ld_o,
                      const float* __restrict__ gw, float eps_g, const float* __restrict__ nw, float eps_bl,
                      int8_t* __restrict__ q, float* __restrict__ dq, int32_t* __restrict__ rowsum, int64_t M, int D) {
    extern __shared__ __align__(16) float sw[];
    constexpr int RPC = FT / RT;                  // rows this CTA works on side by side
    __shared__ RedScratch reds[RPC];
    RedScratch& red = reds[threadIdx.x / RT];
    const int rg = threadIdx.x / RT;
    constexpr int V = 16 / sizeof(T);
    pdl_trigger();
    stage_weights(sw, gw, D);
    stage_weights(sw + D, nw, D);
    pdl_wait();
    __syncthreads();
    // Row loop (LAT = 0): next row by cp.async into thread-private slots, as in prenorm_quant_kernel
    T* sg = reinterpret_cast<T*>(sw + 2 * D) + (size_t)rg * 2 * D;   // per row in flight: [D] g row, [D] o row (LAT = 0 only)
    T* so = sg + D;
    auto fetch = [&](int64_t row) {
        ROW_FOREACH(V, D, it, c) {
            cp_async16(sg + c, gx + row * ld_g + c);
            cp_async16(so + c, o + row * ld_o + c);
        }
        cp_async_commit();
    };
    const int64_t row0 = (int64_t)blockIdx.x * RPC + rg, row_step = (int64_t)gridDim.x * RPC;
    if (LAT == 0 && row0 < M) fetch(row0);
    // a CTA takes rows blockIdx.x (* RPC + its row slot), + gridDim.x (* RPC), ...: with many rows the staged norm weights are reused
    for (int64_t m = row0; m < M; m += row_step) {
        const T* gr = LAT == 0 ? sg : gx + m * ld_g;
        const T* orow = LAT == 0 ? so : o + m * ld_o;
        if (LAT == 0) cp_async_wait_all();
        float gv[P], ov[P];
        double ss = 0.0;
        ROW_FOREACH(V, D, it, c) {
            float a[V], b[V];
            load16<T>(gr + c, a);
            load16<T>(orow + c, b);
    #pragma unroll
            for (int i = 0; i < V; ++i) {
                gv[it * V + i] = a[i];
                ov[it * V + i] = b[i];
                ss += (double)a[i] * (double)a[i];
            }
        }
        if (LAT == 0 && m + row_step < M) fetch(m + row_step);   // this thread's slots have just been read
        gatenorm_tail<T, V, P, RT>(gv, ov, ss, D, eps_g, eps_bl, sw, q, dq, rowsum, M, m, red);
    }
}

// Single-token step of the token mixer for row b (mmfreelm/layers/hgrn_bit.py:113-140 with T = 1):
//   f = round(sigmoid(f_raw)); with lb: f = round(lb + round(round(1-lb)*f));  x = round(silu(i_raw)*round(1-f))
//   h = f*h + x  (fp32 state, updated in place);  o = round(h);  then gatenorm_quant(g_raw, o).
template <typename T, int P, int LAT>
__global__ void __launch_bounds__(FT, LAT)
decode_mix_kernel(const T* __restrict__ ifg, int64_t ld, const T* __restrict__ lb, const uint8_t* __restrict__ mask,
                  float* __restrict__ state, const float* __restrict__ gw, float eps_g, const float* __restrict__ nw, float eps_bl,
                  int8_t* __restrict__ q, float* __restrict__ dq, int32_t* __restrict__ rowsum, int64_t M, int D) {
    extern __shared__ __align__(16) float sw[];   // [3][D]: g_norm weight, BitLinear norm weight, lower bound (as float)
    __shared__ RedScratch red;
    constexpr int V = 16 / sizeof(T);
    constexpr int RT = FT;                        // the whole CTA works on one row
    pdl_trigger();
    stage_weights(sw, gw, D);
    stage_weights(sw + D, nw, D);
    // the lower bounds are constants of the model like the norm weights (derived from parameters only): they are
    // staged before the grid-dependency wait and must not be written by the kernels launched just before this one
    if (lb)
        for (int i = threadIdx.x; i < D; i += FT) sw[2 * D + i] = to_f32(lb[i]);
    pdl_wait();
    __syncthreads();
    const int64_t m = blockIdx.x;
    const T* ir = ifg + m * ld;
    const T* fr = ir + D;
    const T* gr = ir + 2 * D;
    float* st = state + m * (int64_t)D;
    // a padding position (mask 0) contributes no input: i * 0, as `i.mul_(attention_mask)` does; the forget gate still applies
    const bool keep = mask == nullptr || mask[m] != 0;
    float gv[P], ov[P];
    double ss = 0.0;
    ROW_FOREACH(V, D, it, c) {
        float iv[V], fv[V], g8[V];
        load16<T>(ir + c, iv);
        load16<T>(fr + c, fv);
        load16<T>(gr + c, g8);
#pragma unroll
        for (int i = 0; i < V; i += 4) {
            float4 h4 = *reinterpret_cast<const float4*>(st + c + i);
            float hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                float2 xv = raw_gate_floor(make_float2(iv[i + j], iv[i + j + 1])), f = raw_gate_floor(make_float2(fv[i + j], fv[i + j + 1]));
                float2 lbv = make_float2(0.0f, 0.0f), oml = make_float2(1.0f, 1.0f);
                if (lb) {
                    lbv = *reinterpret_cast<const float2*>(&sw[2 * D + c + i + j]);
                    oml = make_float2(round_to<T>(__fsub_rn(1.0f, lbv.x)), round_to<T>(__fsub_rn(1.0f, lbv.y)));
                }
                raw_gate_pair<T>(xv, f, lb != nullptr, lbv, oml);
                if (!keep) xv = make_float2(0.0f, 0.0f);
                hh[j] = fmaf(f.x, hh[j], xv.x);
                hh[j + 1] = fmaf(f.y, hh[j + 1], xv.y);
                ov[it * V + i + j] = round_to<T>(hh[j]);
                ov[it * V + i + j + 1] = round_to<T>(hh[j + 1]);
            }
            *reinterpret_cast<float4*>(st + c + i) = make_float4(hh[0], hh[1], hh[2], hh[3]);
        }
#pragma unroll
        for (int i = 0; i < V; ++i) {
            gv[it * V + i] = g8[i];
            ss += (double)g8[i] * (double)g8[i];
        }
    }
    gatenorm_tail<T, V, P>(gv, ov, ss, D, eps_g, eps_bl, sw, q, dq, rowsum, M, m, red);
}

// z = round_T(silu(gate)*up), then BitLinear prologue.  gate/up are the two halves of a [M, 2D] tensor.
template <typename T, int P, int LAT, int RT = FT>
__global__ void __launch_bounds__(FT, LAT)
swiglu_quant_kernel(const T* __restrict__ gate, const T* __restrict__ up, int64_t ld, const float* __restrict__ nw,
                    float eps_bl, int8_t* __restrict__ q, float* __restrict__ dq, int32_t* __restrict__ rowsum, int64_t M, int D) {
    extern __shared__ __align__(16) float sw[];
    constexpr int RPC = FT / RT;                  // rows this CTA works on side by side
    __shared__ RedScratch reds[RPC];
    RedScratch& red = reds[threadIdx.x / RT];
    const int rg = threadIdx.x / RT;
    constexpr int V = 16 / sizeof(T);
    pdl_trigger();
    stage_weights(sw, nw, D);
    pdl_wait();
    __syncthreads();
    // Row loop (LAT = 0): the next row of this CTA travels global -> shared memory by cp.async while the current one is
    // reduced and quantised, so its load latency is hidden without holding it in registers.  Every thread copies and
    // later reads the same 16-byte slots, so the copies need no barrier, only the thread's own wait.
    T* sg = reinterpret_cast<T*>(sw + D) + (size_t)rg * 2 * D;   // per row in flight: [D] gate row, [D] up row (LAT = 0 only)
    T* su = sg + D;
    auto fetch = [&](int64_t row) {
        ROW_FOREACH(V, D, it, c) {
            cp_async16(sg + c, gate + row * ld + c);
            cp_async16(su + c, up + row * ld + c);
        }
        cp_async_commit();
    };
    const int64_t row0 = (int64_t)blockIdx.x * RPC + rg, row_step = (int64_t)gridDim.x * RPC;
    if (LAT == 0 && row0 < M) fetch(row0);
    // a CTA takes rows blockIdx.x (* RPC + its row slot), + gridDim.x (* RPC), ...: with many rows the staged norm weights are reused
    for (int64_t m = row0; m < M; m += row_step) {
        const T* gr = LAT == 0 ? sg : gate + m * ld;
        const T* ur = LAT == 0 ? su : up + m * ld;
        if (LAT == 0) cp_async_wait_all();
        float v[P];
        double ss = 0.0;
        ROW_FOREACH(V, D, it, c) {
            float gv[V], uv[V];
            load16<T>(gr + c, gv);
            load16<T>(ur + c, uv);
    #pragma unroll
            for (int i = 0; i < V; i += 2) {
                const float2 t = silu_mul2(make_float2(gv[i], gv[i + 1]), make_float2(uv[i], uv[i + 1]));
                gv[i] = t.x;
                gv[i + 1] = t.y;
            }
            uint32_t bits[V / 2];
            round_vec<T, V>(gv, bits);
    #pragma unroll
            for (int i = 0; i < V; ++i) v[it * V + i] = gv[i];
            sumsq_rounded<T, V>(gv, bits, ss);
        }
        if (LAT == 0 && m + row_step < M) fetch(m + row_step);   // this thread's slots have just been read
        bitlinear_prologue<V, 1, P, RT>(v, D, ss, eps_bl, sw, q, dq, rowsum, M, m, red);
    }
}

}  // namespace

// =========================================================================================================
// C ABI
// =========================================================================================================
#define FUSED_ROW_CHECKS(name, D)                                                                                   \
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, name ": unknown dtype %d", dtype);                             \
    MMF_REQUIRE(M >= 0 && (D) > 0 && (D) <= MAX_D && (D) % 16 == 0, MMF_ERR_BAD_SHAPE,                               \
                name ": need 0 < D <= 8192 and D %% 16 == 0 (D=%lld)", (long long)(D));

// CTAs of `kernel` (FT threads, `smem` dynamic bytes) that fit on one SM at a time; asked of the runtime once per
// (kernel, smem) and remembered per host thread
static int resident_ctas(const void* kernel, size_t smem) {
    struct Entry { const void* k; size_t s; int occ; };
    thread_local Entry cache[64];
    thread_local int n = 0;
    for (int i = 0; i < n; ++i)
        if (cache[i].k == kernel && cache[i].s == smem) return cache[i].occ;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, FT, smem) != cudaSuccess || occ < 1) {
        (void)cudaGetLastError();
        occ = 4;
    }
    if (n < 64) cache[n++] = Entry{kernel, smem, occ};
    return occ;
}
// one CTA per row while all of them are resident at once; beyond that exactly one resident set of CTAs, which loop
// over the rows (a partial second wave would leave SMs idle at the end)
template <typename Kern>
static inline unsigned row_grid(Kern kernel, size_t smem, int64_t M, int rows_per_cta = 1) {
    const int64_t cap = (int64_t)148 * resident_ctas(reinterpret_cast<const void*>(kernel), smem);
    const int64_t want = (M + rows_per_cta - 1) / rows_per_cta;
    return (unsigned)(want < cap ? want : cap);
}
// Prompt-sized calls (MMF_FOUR_ROWS_MIN_M rows and more): four rows per CTA with 64 threads each for rows of at most 2048
// values, two rows with 128 threads each up to 4096 values.  A thread then holds up to 32 values of its row instead of
// 8 - 16, so the reductions of a row (two fp64 sums, the absmax, the code sum: a fifth of all instructions at 8 values
// per thread) cost a quarter (half) per value, and a row's threads meet at a barrier of 64 (128) instead of 256.
// Measured at 32768 rows of 2048 values: 220 -> 160 us (three projections), 150 -> 89 us (one), 150 -> 104 us (gate norm).
constexpr int ROW_QUARTER = 64, ROW_HALF = 128;
// run `...` with RT bound to the threads per row of a prompt-sized call on rows of D values (D <= ROW_HALF * MAX_PER)
#define FUSED_DISPATCH_RT(D, RT, ...)                                              \
    if ((D) <= ROW_QUARTER * MAX_PER) { constexpr int RT = ROW_QUARTER; __VA_ARGS__; } \
    else { constexpr int RT = ROW_HALF; __VA_ARGS__; }
#ifndef MMF_FOUR_ROWS_MIN_M
#define MMF_FOUR_ROWS_MIN_M 3072
#endif

// Run `...` with `P` (row values per thread) bound to the smallest compiled size that holds a row of D values.
#define FUSED_DISPATCH_P(D, P, ...)                                   \
    if ((D) <= FT * 8) { constexpr int P = 8; __VA_ARGS__; }          \
    else if ((D) <= FT * 16) { constexpr int P = 16; __VA_ARGS__; }   \
    else if ((D) <= FT * 24) { constexpr int P = 24; __VA_ARGS__; }   \
    else { constexpr int P = 32; __VA_ARGS__; }

// Two builds of every kernel.  LAT = 1 (at least one CTA per SM: the compiler may spend registers on overlapping the
// loads and reductions of a row) for calls whose rows are all resident at once, i.e. decode steps, where the latency of
// a row is what counts; LAT = 0 (no hint: fewer registers, more resident CTAs) for the row loop over a prompt.
// Measured on whole decode steps: the register-rich build still wins at 320 - 448 rows (2 - 3 %), equal at 512.
#ifndef MMF_LAT_MAX_ROWS
#define MMF_LAT_MAX_ROWS 592
#endif
constexpr int64_t LAT_MAX_ROWS = MMF_LAT_MAX_ROWS;
#define FUSED_DISPATCH_LAT(M, LAT, ...)                                \
    if ((M) <= LAT_MAX_ROWS) { constexpr int LAT = 1; __VA_ARGS__; }   \
    else { constexpr int LAT = 0; __VA_ARGS__; }

// the 48 KB that need no opt-in include the kernel's static shared memory (reduction scratch)
#define FUSED_SMEM_ATTR(kernel, smem) \
    if ((smem) + 2048 > 48 * 1024) MMF_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(smem)))

#ifdef MMF_EXPERIMENTS
static long long* g_row_trace = nullptr;
// experiments build only: device buffer ([0] = launch counter, records of 8 stamps from word 8 on) or NULL to switch off
extern "C" int mmf_row_trace(long long* buffer_dev) { g_row_trace = buffer_dev; return MMF_OK; }
#endif

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
                    (!residual_out || mmf_aligned(residual_out, 16)) && (!y_out || mmf_aligned(y_out, 16)) && (!q || mmf_aligned(q, 16)) &&
                    mmf_aligned(norm_w, 16) && mmf_aligned(nw0, 16) && mmf_aligned(nw1, 16) && mmf_aligned(nw2, 16),
                MMF_ERR_ALIGN, "mmf_prenorm_quant: rows and norm weights must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    PrenormArgs a;
    a.x = x; a.ld_x = ld_x; a.res = residual; a.ld_res = ld_res; a.res_out = residual_out; a.y_out = y_out;
    a.norm_w = norm_w; a.eps_norm = eps_norm; a.nws[0] = nw0; a.nws[1] = nw1; a.nws[2] = nw2; a.eps_bl = eps_bl;
    a.q = q; a.dq = dq; a.rowsum = rowsum; a.M = M; a.D = (int)D; a.G = groups; a.round_sum_first = round_sum_first;
    // decode-sized call with three projections: one CTA per (row, projection).  The shared statistics are recomputed
    // by each of the three CTAs (same loads, same operations, same results), the three quantisation passes run side by
    // side: measured 1.5 us -> 0.8 us of prologue after the grid dependency resolves
    a.gsplit = groups == 3 && M <= 128 ? 1 : 0;
#ifdef MMF_EXPERIMENTS
    a.trace = g_row_trace;
#endif
    if (M >= MMF_FOUR_ROWS_MIN_M && D <= ROW_HALF * MAX_PER && !a.gsplit) {
        MMF_DISPATCH(dtype, T, { FUSED_DISPATCH_RT(D, RT, {
            constexpr int P = MAX_PER, RPC = FT / RT;
            const size_t smem = (size_t)(1 + groups) * D * sizeof(float) + (size_t)RPC * 2 * D * sizeof(T);   // + row staging
            FUSED_SMEM_ATTR((prenorm_quant_kernel<T, P, 0, RT>), smem);
            const dim3 grid(row_grid(prenorm_quant_kernel<T, P, 0, RT>, smem, M, RPC));
            MMF_CUDA(mmf_launch_pdl(prenorm_quant_kernel<T, P, 0, RT>, grid, dim3(FT), smem, (cudaStream_t)stream, a));
        }); });
        MMF_LAUNCH_CHECK("prenorm_quant_kernel");
        return MMF_OK;
    }
    MMF_DISPATCH(dtype, T, {
        FUSED_DISPATCH_P(D, P, { FUSED_DISPATCH_LAT(M, LAT, {
            const size_t smem = (size_t)(1 + (a.gsplit ? 1 : groups)) * D * sizeof(float) + (LAT ? 0 : (size_t)2 * D * sizeof(T));   // + row staging
            FUSED_SMEM_ATTR((prenorm_quant_kernel<T, P, LAT>), smem);
            const dim3 grid(a.gsplit ? (unsigned)M : row_grid(prenorm_quant_kernel<T, P, LAT>, smem, M), a.gsplit ? 3u : 1u);
            MMF_CUDA(mmf_launch_pdl(prenorm_quant_kernel<T, P, LAT>, grid, dim3(FT), smem, (cudaStream_t)stream, a));
        }); });
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
    MMF_REQUIRE(mmf_aligned(g, 16) && mmf_aligned(o, 16) && mmf_aligned(q, 16) && (ld_g * es) % 16 == 0 && (ld_o * es) % 16 == 0 &&
                    mmf_aligned(gnorm_w, 16) && mmf_aligned(nw, 16),
                MMF_ERR_ALIGN, "mmf_gatenorm_quant: rows and norm weights must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    if (M >= MMF_FOUR_ROWS_MIN_M && D <= ROW_HALF * MAX_PER) {
        MMF_DISPATCH(dtype, T, { FUSED_DISPATCH_RT(D, RT, {
            constexpr int P = MAX_PER, RPC = FT / RT;
            const size_t smem = (size_t)2 * D * sizeof(float) + (size_t)RPC * 2 * D * sizeof(T);   // + row staging
            FUSED_SMEM_ATTR((gatenorm_quant_kernel<T, P, 0, RT>), smem);
            MMF_CUDA(mmf_launch_pdl(gatenorm_quant_kernel<T, P, 0, RT>, dim3(row_grid(gatenorm_quant_kernel<T, P, 0, RT>, smem, M, RPC)),
                                    dim3(FT), smem, (cudaStream_t)stream, (const T*)g, ld_g, (const T*)o, ld_o, gnorm_w, eps_g, nw, eps_bl, q, dq,
                                    rowsum, M, (int)D));
        }); });
        MMF_LAUNCH_CHECK("gatenorm_quant_kernel");
        return MMF_OK;
    }
    MMF_DISPATCH(dtype, T, {
        FUSED_DISPATCH_P(D, P, { FUSED_DISPATCH_LAT(M, LAT, {
            const size_t smem = (size_t)2 * D * sizeof(float) + (LAT ? 0 : (size_t)2 * D * sizeof(T));   // + row staging
            FUSED_SMEM_ATTR((gatenorm_quant_kernel<T, P, LAT>), smem);
            MMF_CUDA(mmf_launch_pdl(gatenorm_quant_kernel<T, P, LAT>, dim3(row_grid(gatenorm_quant_kernel<T, P, LAT>, smem, M)), dim3(FT), smem, (cudaStream_t)stream, (const T*)g,
                                    ld_g, (const T*)o, ld_o, gnorm_w, eps_g, nw, eps_bl, q, dq, rowsum, M, (int)D));
        }); });
    });
    MMF_LAUNCH_CHECK("gatenorm_quant_kernel");
    return MMF_OK;
}

extern "C" int mmf_decode_mix(const void* ifg, int64_t ld, int dtype, const void* lower_bound, float* state,
                              const float* gnorm_w, float eps_g, const float* nw, float eps_bl, int8_t* q, float* dq,
                              int32_t* rowsum, int64_t M, int64_t D, void* stream) {
    return mmf_decode_mix_masked(ifg, ld, dtype, lower_bound, nullptr, state, gnorm_w, eps_g, nw, eps_bl, q, dq, rowsum, M, D, stream);
}

extern "C" int mmf_decode_mix_masked(const void* ifg, int64_t ld, int dtype, const void* lower_bound, const uint8_t* mask,
                                     float* state, const float* gnorm_w, float eps_g, const float* nw, float eps_bl,
                                     int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(ifg && state && q && dq && rowsum, MMF_ERR_BAD_ARG, "mmf_decode_mix: null pointer");
    FUSED_ROW_CHECKS("mmf_decode_mix", D);
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(ld >= 3 * D, MMF_ERR_BAD_SHAPE, "mmf_decode_mix: ld must cover the three projections");
    MMF_REQUIRE(mmf_aligned(ifg, 16) && (ld * es) % 16 == 0 && mmf_aligned(state, 16) && mmf_aligned(q, 16) &&
                    mmf_aligned(gnorm_w, 16) && mmf_aligned(nw, 16),
                MMF_ERR_ALIGN, "mmf_decode_mix: rows, state and norm weights must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    const size_t smem = (size_t)3 * D * sizeof(float);
    MMF_DISPATCH(dtype, T, {
        FUSED_DISPATCH_P(D, P, { FUSED_DISPATCH_LAT(M, LAT, {
            FUSED_SMEM_ATTR((decode_mix_kernel<T, P, LAT>), smem);
            MMF_CUDA(mmf_launch_pdl(decode_mix_kernel<T, P, LAT>, dim3((unsigned)M), dim3(FT), smem, (cudaStream_t)stream, (const T*)ifg, ld,
                                    (const T*)lower_bound, mask, state, gnorm_w, eps_g, nw, eps_bl, q, dq, rowsum, M, (int)D));
        }); });
    });
    MMF_LAUNCH_CHECK("decode_mix_kernel");
    return MMF_OK;
}

extern "C" int mmf_swiglu_quant(const void* gate, const void* up, int64_t ld, int dtype, const float* nw, float eps_bl,
                                int8_t* q, float* dq, int32_t* rowsum, int64_t M, int64_t D, void* stream) {
    MMF_REQUIRE(gate && up && q && dq && rowsum, MMF_ERR_BAD_ARG, "mmf_swiglu_quant: null pointer");
    FUSED_ROW_CHECKS("mmf_swiglu_quant", D);
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(gate, 16) && mmf_aligned(up, 16) && mmf_aligned(q, 16) && (ld * es) % 16 == 0 && mmf_aligned(nw, 16),
                MMF_ERR_ALIGN, "mmf_swiglu_quant: rows and norm weight must be 16-byte aligned");
    if (M == 0) return MMF_OK;
    // prompt-sized calls: rows side by side in one CTA as in mmf_prenorm_quant; a row of the MLP width (5632, 6912) takes
    // two rows per CTA with 128 threads and up to 56 values per thread each
#define SWIGLU_ROWS(RT, P)                                                                                                        \
    MMF_DISPATCH(dtype, T, {                                                                                                      \
        constexpr int RPC = FT / (RT);                                                                                            \
        const size_t smem = (size_t)D * sizeof(float) + (size_t)RPC * 2 * D * sizeof(T);                                          \
        FUSED_SMEM_ATTR((swiglu_quant_kernel<T, P, 0, RT>), smem);                                                                \
        MMF_CUDA(mmf_launch_pdl(swiglu_quant_kernel<T, P, 0, RT>, dim3(row_grid(swiglu_quant_kernel<T, P, 0, RT>, smem, M, RPC)),  \
                                dim3(FT), smem, (cudaStream_t)stream, (const T*)gate, (const T*)up, ld, nw, eps_bl, q, dq, rowsum, M, \
                                (int)D));                                                                                         \
    });                                                                                                                           \
    MMF_LAUNCH_CHECK("swiglu_quant_kernel");                                                                                      \
    return MMF_OK
    if (M >= MMF_FOUR_ROWS_MIN_M && D <= ROW_HALF * 56) {
        if (D <= ROW_QUARTER * MAX_PER) { SWIGLU_ROWS(ROW_QUARTER, MAX_PER); }
        if (D <= ROW_HALF * MAX_PER) { SWIGLU_ROWS(ROW_HALF, MAX_PER); }
        SWIGLU_ROWS(ROW_HALF, 56);
    }
#undef SWIGLU_ROWS
    MMF_DISPATCH(dtype, T, {
        FUSED_DISPATCH_P(D, P, { FUSED_DISPATCH_LAT(M, LAT, {
            const size_t smem = (size_t)D * sizeof(float) + (LAT ? 0 : (size_t)2 * D * sizeof(T));   // + row staging in the row loop
            FUSED_SMEM_ATTR((swiglu_quant_kernel<T, P, LAT>), smem);
            MMF_CUDA(mmf_launch_pdl(swiglu_quant_kernel<T, P, LAT>, dim3(row_grid(swiglu_quant_kernel<T, P, LAT>, smem, M)), dim3(FT), smem, (cudaStream_t)stream, (const T*)gate,
                                    (const T*)up, ld, nw, eps_bl, q, dq, rowsum, M, (int)D));
        }); });
    });
    MMF_LAUNCH_CHECK("swiglu_quant_kernel");
    return MMF_OK;
}
