// HGRN recurrence h_t = f_t * h_{t-1} + x_t as an HBM-bound streaming scan.
//
// Work decomposition: one CTA owns 64 channels of one sequence and one chunk of the time axis.
// [64 timesteps x 64 channels] tiles of x and g arrive in shared memory by tiled TMA (one elected
// thread issues them, a 2- or 3-deep ring of mbarrier-tracked stages) and the output tile leaves by a
// TMA store from a double-buffered shared-memory tile, so no thread spends instructions on addressing
// or copying global memory and x, g, o are each touched exactly once (8 B per element for bf16 x/o
// and an fp32 gate, 6 B with the 16-bit raw gate).  Inside a stage warp `sub` scans timesteps
// [8*sub, 8*sub+8) of all 64 channels from a zero state — lane = channel pair, packed 2-element
// shared-memory accesses — and the eight sub-chunk aggregates (gate product, local end state) meet in
// shared memory: every thread folds the ones before it and the carry of the previous stage into its
// carry-in and fixes its eight states up, h_t = h_local_t + prod_t * carry (fp32 throughout).
// With a 16-bit gate a CTA holds 48 KB and four of them share an SM (two with an fp32 gate).  Halving the CTA
// (32 timesteps, 4 warps, eight per SM) to spread a 512-CTA grid more evenly was measured and is 40 % slower.
//
// When B*D/64 CTAs would leave most SMs idle the time axis is split into NT chunks
// ("chunked parallel scan"): pass 1 reduces every chunk but the last to its aggregate
// (prod f, local end state), pass 2 lets each chunk fold the aggregates before it into its
// carry-in and scans.  Pass 1 re-reads x and g, so it is only used when it buys occupancy.
#include "common.cuh"
#include "tensor_map.cuh"

namespace {

constexpr int HG_BD = 64;       // channels per CTA
constexpr int HG_TS = 64;       // timesteps per stage
constexpr int HG_SUB = 8;       // sub-chunks (warps) per stage
constexpr int HG_SUBT = HG_TS / HG_SUB;   // timesteps per thread and stage
constexpr int HG_THREADS = (HG_BD / 2) * HG_SUB;
// TMA ring depth: two stages when x and g are both 16-bit (the raw projections inside the model), three when the gate is fp32
template <typename TX, typename TG> struct HgStages { static constexpr int value = sizeof(TX) + sizeof(TG) <= 4 ? 2 : 3; };
constexpr long long HG_WAIT_LIMIT = 2000000000ll;   // clock cycles (about a second) before a wait gives up

__device__ int g_hgrn_wait_failed = 0;   // set when a bounded wait on a TMA stage gave up

__device__ __forceinline__ uint32_t hg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void hg_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(hg_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void hg_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(hg_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool hg_mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred P1;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, P1;\n\t}"
        : "=r"(ok)
        : "r"(hg_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded: returns false (and raises *abort_flag) if the phase does not complete within HG_WAIT_LIMIT cycles
__device__ __forceinline__ bool hg_mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (hg_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (hg_mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > HG_WAIT_LIMIT) {
            *abort_flag = 1;
            return false;
        }
    }
}
__device__ __forceinline__ void hg_tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(hg_smem_u32(dst)), "l"(map), "r"(hg_smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void hg_tma_store_3d(const CUtensorMap* map, const void* src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(hg_smem_u32(src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void hg_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void hg_bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void hg_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void hg_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// two adjacent elements <-> float2
__device__ __forceinline__ float2 ld2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 ld2(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ float2 ld2(const __half* p) { return __half22float2(*reinterpret_cast<const __half2*>(p)); }
__device__ __forceinline__ void st2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void st2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
__device__ __forceinline__ void st2(__half* p, float a, float b) { *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b); }

// exp(v) for v <= 0 (a log forget gate): ex2.approx of the rounded product plus a first-order correction with
// the product's rounding residual, so that the relative error stays at the 2^-22 of the approximation itself
__device__ __forceinline__ float exp_gate(float v) {
    const float L2E = 1.4426950408889634f;
    const float t = __fmul_rn(v, L2E);
    const float e = __fmaf_rn(v, L2E, -t);
    float p;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(t));
    return __fmaf_rn(__fmul_rn(p, 0.6931471805599453f), e, p);
}

template <typename T> __device__ __forceinline__ float load_state(const void* p, int64_t i) {
    return to_f32(reinterpret_cast<const T*>(p)[i]);
}
__device__ __forceinline__ float load_state_dt(const void* p, int64_t i, int dt) {
    return dt == MMF_F32 ? load_state<float>(p, i) : dt == MMF_BF16 ? load_state<__nv_bfloat16>(p, i)
                                                                     : load_state<__half>(p, i);
}
__device__ __forceinline__ void store_state_dt(void* p, int64_t i, int dt, float v) {
    if (dt == MMF_F32) reinterpret_cast<float*>(p)[i] = v;
    else if (dt == MMF_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// workspace layout (floats): h0 copy [B,D] | prod_f [B,NT,D] | h_loc [B,NT,D]
struct HgrnWs {
    float* h0c;
    float* agg_a;
    float* agg_h;
};

// gate conventions
constexpr int HG_LINEAR = 0;  // g is the forget gate itself           (fused_recurrent_hgrn)
constexpr int HG_LOG = 1;     // g is its logarithm                     (chunk_hgrn)
constexpr int HG_RAW = 2;     // x, g are the raw i/f projection outputs (HGRNBitAttention's gate math fused in):
                              //   f = round(sigmoid(g)); with a lower bound lb: f = round(lb + round(round(1-lb)*f))
                              //   x = round(silu(x_raw) * round(1-f));  every round() is to the activation dtype TX

// load of a raw projection pair: in raw mode limited from below (on the packed pair for a 16-bit dtype)
template <int MODE> __device__ __forceinline__ float2 ld2g(const float* p) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    return MODE == 2 ? raw_gate_floor(v) : v;
}
template <int MODE> __device__ __forceinline__ float2 ld2g(const __nv_bfloat16* p) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
    return unpack2(MODE == 2 ? raw_gate_floor(v) : v);
}
template <int MODE> __device__ __forceinline__ float2 ld2g(const __half* p) {
    const __half2 v = *reinterpret_cast<const __half2*>(p);
    return unpack2(MODE == 2 ? raw_gate_floor(v) : v);
}

// raw (x, g) of a channel pair -> (x_t, f_t) of the recurrence
template <typename TX, int MODE>
__device__ __forceinline__ void gate_transform2(float2& xv, float2& f, bool has_lb, float2 lbv, float2 oml) {
    if (MODE == HG_LOG) { f.x = exp_gate(f.x); f.y = exp_gate(f.y); }
    if (MODE == HG_RAW) raw_gate_pair<TX>(xv, f, has_lb, lbv, oml);
}

// AGG = true : pass 1, chunks 0..NT-2 -> aggregates (no o written)
// AGG = false: pass 2 (or the only pass when NT == 1) -> o, ht
// Tensor maps: x, g, o as [B][T][D] with box [1][HG_TS][64]; rows past T read as zero and are not stored, channels
// past D likewise.  chunk_len is a multiple of HG_TS, so only the last stage of the last chunk can be partial.
template <typename TX, typename TG, int MODE, bool AGG>
__global__ void __launch_bounds__(HG_THREADS, 4)
hgrn_scan_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap g_map,
                 const __grid_constant__ CUtensorMap o_map, const TX* __restrict__ lb, const uint8_t* __restrict__ mask,
                 const void* __restrict__ h0, void* __restrict__ ht, int state_dt, int T, int D, int NT, int chunk_len,
                 HgrnWs ws) {
    pdl_trigger();
    if (threadIdx.x == 0) {   // descriptors into the descriptor cache before the dependency wait ends
        asm volatile("prefetch.tensormap [%0];" ::"l"(&x_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&g_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&o_map) : "memory");
    }
    extern __shared__ uint8_t smem_dyn[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 127) & ~uintptr_t(127));
    constexpr int HG_STAGES = HgStages<TX, TG>::value;
    constexpr int XB = HG_TS * HG_BD * sizeof(TX);  // bytes of one x stage (= one output tile)
    constexpr int GB = HG_TS * HG_BD * sizeof(TG);
    TX* sx = reinterpret_cast<TX*>(smem);
    TG* sg = reinterpret_cast<TG*>(smem + HG_STAGES * XB);
    TX* so = reinterpret_cast<TX*>(smem + HG_STAGES * (XB + GB));       // two output tiles
    __shared__ float s_agg_a[HG_SUB][HG_BD], s_agg_h[HG_SUB][HG_BD];
    __shared__ float s_carry[2][HG_BD];          // carry of the previous stage, double-buffered by stage parity
    __shared__ __align__(8) uint64_t s_full[HG_STAGES];
    __shared__ int s_abort;

    const int d0 = blockIdx.x * HG_BD;
    const int c = blockIdx.y;
    const int b = blockIdx.z;
    const int tid = threadIdx.x;
    const int lc = (tid & 31) * 2;               // first of this thread's two channels inside the block
    const int sub = tid >> 5;                    // warp = sub-chunk of the stage
    const int ch = d0 + lc;
    const bool ch_ok = ch < D;                   // D is even: both channels of the pair are in or out together
    const int t_begin = c * chunk_len;
    const int nsteps = min(T, t_begin + chunk_len) - t_begin;            // <= 0: an empty chunk (identity)
    const int nstage = nsteps > 0 ? (nsteps + HG_TS - 1) / HG_TS : 0;
    volatile int* abort_flag = &s_abort;

    if (tid == 0) {
        for (int i = 0; i < HG_STAGES; ++i) hg_mbar_init(&s_full[i], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();                                  // x and g are the preceding kernel's output

    auto issue = [&](int s) {                    // thread 0 only
        if (s < nstage) {
            const int buf = s % HG_STAGES;
            hg_mbar_expect_tx(&s_full[buf], (uint32_t)(XB + GB));
            hg_tma_load_3d(sx + buf * HG_TS * HG_BD, &x_map, &s_full[buf], d0, t_begin + s * HG_TS, b);
            hg_tma_load_3d(sg + buf * HG_TS * HG_BD, &g_map, &s_full[buf], d0, t_begin + s * HG_TS, b);
        }
    };
    if (tid == 0)
        for (int s = 0; s < HG_STAGES; ++s) issue(s);

    const bool has_lb = MODE == HG_RAW && lb != nullptr;      // uniform over the kernel
    float2 lbv = make_float2(0.0f, 0.0f), oml = make_float2(1.0f, 1.0f);
    if (has_lb && ch_ok) {
        lbv = ld2(lb + ch);
        oml.x = round_to<TX>(__fsub_rn(1.0f, lbv.x));
        oml.y = round_to<TX>(__fsub_rn(1.0f, lbv.y));
    }
    // carry into the first stage
    if (sub == 0) {
        float hc[2] = {0.0f, 0.0f};
        if (!AGG && ch_ok) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int64_t sidx = (int64_t)b * D + ch + k;
                if (NT == 1) {
                    if (h0) hc[k] = load_state_dt(h0, sidx, state_dt);
                } else {
                    float h = ws.h0c[sidx];
                    for (int j = 0; j < c; ++j) {
                        const int64_t i = ((int64_t)b * NT + j) * (int64_t)D + ch + k;
                        h = fmaf(ws.agg_a[i], h, ws.agg_h[i]);
                    }
                    hc[k] = h;
                }
            }
        }
        s_carry[0][lc] = hc[0];
        s_carry[0][lc + 1] = hc[1];
        if (AGG && c == 0 && ch_ok) {
#pragma unroll
            for (int k = 0; k < 2; ++k)
                ws.h0c[(int64_t)b * D + ch + k] = h0 ? load_state_dt(h0, (int64_t)b * D + ch + k, state_dt) : 0.0f;
        }
    }
    float2 a_run = make_float2(1.0f, 1.0f);   // AGG: product of all gates of this chunk

    for (int s = 0; s < nstage; ++s) {
        const int buf = s % HG_STAGES;
        hg_mbar_wait(&s_full[buf], (uint32_t)((s / HG_STAGES) & 1), abort_flag);
        const int rows = min(HG_TS, nsteps - s * HG_TS);
        float2 hl[HG_SUBT], ap[HG_SUBT];
        {
            const TX* px = sx + (buf * HG_TS + sub * HG_SUBT) * HG_BD + lc;
            const TG* pg = sg + (buf * HG_TS + sub * HG_SUBT) * HG_BD + lc;
            float2 h = make_float2(0.0f, 0.0f), a = make_float2(1.0f, 1.0f);
            // padding mask of the sequence (attention layer only): a masked position contributes no input
            const uint8_t* pm = mask ? mask + (int64_t)b * T + t_begin + s * HG_TS + sub * HG_SUBT : nullptr;
            if (rows == HG_TS) {
#pragma unroll
                for (int j = 0; j < HG_SUBT; ++j) {
                    float2 xv = ld2g<MODE>(px + j * HG_BD), f = ld2g<MODE>(pg + j * HG_BD);
                    gate_transform2<TX, MODE>(xv, f, has_lb, lbv, oml);
                    if (pm && !pm[j]) xv = make_float2(0.0f, 0.0f);
                    h = __ffma2_rn(f, h, xv);      // both channels in one packed f32x2 instruction
                    a = __fmul2_rn(a, f);
                    hl[j] = h; ap[j] = a;
                }
            } else {
#pragma unroll
                for (int j = 0; j < HG_SUBT; ++j) {
                    float2 xv = ld2g<MODE>(px + j * HG_BD), f = ld2g<MODE>(pg + j * HG_BD);
                    gate_transform2<TX, MODE>(xv, f, has_lb, lbv, oml);
                    if (sub * HG_SUBT + j >= rows) {   // steps past the end of the sequence are the identity
                        xv = make_float2(0.0f, 0.0f);
                        f = make_float2(1.0f, 1.0f);
                    } else if (pm && !pm[j]) {
                        xv = make_float2(0.0f, 0.0f);
                    }
                    h = __ffma2_rn(f, h, xv);      // both channels in one packed f32x2 instruction
                    a = __fmul2_rn(a, f);
                    hl[j] = h; ap[j] = a;
                }
            }
            *reinterpret_cast<float2*>(&s_agg_a[sub][lc]) = a;
            *reinterpret_cast<float2*>(&s_agg_h[sub][lc]) = h;
        }
        // the output tile written two stages ago must have been read by its TMA store before it is reused
        if (!AGG && tid == 0) hg_bulk_wait_read<1>();
        __syncthreads();                          // aggregates visible; all reads of stage buffer `buf` are done
        if (*abort_flag) break;                   // uniform: written before the barrier
        if (tid == 0) issue(s + HG_STAGES);       // refill the stage just consumed
        // carry-in of this thread's sub-chunk: previous stage's carry folded through the sub-chunks before it
        float2 cin = *reinterpret_cast<const float2*>(&s_carry[s & 1][lc]);
#pragma unroll
        for (int q = 0; q < HG_SUB - 1; ++q) {
            if (q < sub) {                        // warp-uniform
                const float2 qa = *reinterpret_cast<const float2*>(&s_agg_a[q][lc]);
                const float2 qh = *reinterpret_cast<const float2*>(&s_agg_h[q][lc]);
                cin = __ffma2_rn(qa, cin, qh);
            }
        }
        if (AGG) {
            if (sub == 0) {
#pragma unroll
                for (int q = 0; q < HG_SUB; ++q) {
                    const float2 qa = *reinterpret_cast<const float2*>(&s_agg_a[q][lc]);
                    a_run.x *= qa.x; a_run.y *= qa.y;
                }
            }
        } else {
            TX* po = so + ((s & 1) * HG_TS + sub * HG_SUBT) * HG_BD + lc;
#pragma unroll
            for (int j = 0; j < HG_SUBT; ++j) {
                const float2 o2 = __ffma2_rn(ap[j], cin, hl[j]);
                st2(po + j * HG_BD, o2.x, o2.y);
            }
            hg_fence_async_smem();                // generic-proxy writes -> visible to the TMA store
        }
        if (sub == HG_SUB - 1) {
            s_carry[(s + 1) & 1][lc] = fmaf(ap[HG_SUBT - 1].x, cin.x, hl[HG_SUBT - 1].x);
            s_carry[(s + 1) & 1][lc + 1] = fmaf(ap[HG_SUBT - 1].y, cin.y, hl[HG_SUBT - 1].y);
        }
        __syncthreads();                          // output tile and next carry complete; aggregates may be overwritten
        if (!AGG && tid == 0) {
            hg_tma_store_3d(&o_map, so + (s & 1) * HG_TS * HG_BD, d0, t_begin + s * HG_TS, b);
            hg_bulk_commit();
        }
    }
    if (!AGG && tid == 0) hg_bulk_wait_all();     // shared memory must outlive the stores that read it
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) atomicExch(&g_hgrn_wait_failed, 1);
        return;
    }

    if (ch_ok && sub == 0) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float h_end = s_carry[nstage & 1][lc + k];
            if (AGG) {
                const int64_t i = ((int64_t)b * NT + c) * (int64_t)D + ch + k;
                ws.agg_a[i] = k ? a_run.y : a_run.x;
                ws.agg_h[i] = h_end;
            } else if (ht && c == NT - 1) {
                store_state_dt(ht, (int64_t)b * D + ch + k, state_dt, h_end);
            }
        }
    }
}

// T = 1 (a decode step outside the fused chain): one thread per channel pair, h = f * h0 + x, o = h, state written back.
template <typename TX, typename TG, int MODE>
__global__ void __launch_bounds__(256)
hgrn_step_kernel(const TX* __restrict__ x, int64_t ld_x, const TG* __restrict__ g, int64_t ld_g, const TX* __restrict__ lb,
                 const uint8_t* __restrict__ mask, const void* __restrict__ h0, void* __restrict__ ht, int state_dt,
                 TX* __restrict__ o, int64_t B, int D) {
    pdl_trigger();
    pdl_wait();
    const int64_t idx = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (idx >= B * D) return;
    const int64_t b = idx / D;
    const int ch = (int)(idx - b * D);
    float2 xv = ld2g<MODE>(x + b * ld_x + ch), f = ld2g<MODE>(g + b * ld_g + ch);
    const bool has_lb = MODE == HG_RAW && lb != nullptr;
    float2 lbv = make_float2(0.0f, 0.0f), oml = make_float2(1.0f, 1.0f);
    if (has_lb) {
        lbv = ld2(lb + ch);
        oml.x = round_to<TX>(__fsub_rn(1.0f, lbv.x));
        oml.y = round_to<TX>(__fsub_rn(1.0f, lbv.y));
    }
    gate_transform2<TX, MODE>(xv, f, has_lb, lbv, oml);
    if (mask && !mask[b]) xv = make_float2(0.0f, 0.0f);
    float h0x = 0.0f, h0y = 0.0f;
    if (h0) {
        h0x = load_state_dt(h0, idx, state_dt);
        h0y = load_state_dt(h0, idx + 1, state_dt);
    }
    const float hx = fmaf(f.x, h0x, xv.x), hy = fmaf(f.y, h0y, xv.y);
    st2(o + idx, hx, hy);
    if (ht) {
        store_state_dt(ht, idx, state_dt, hx);
        store_state_dt(ht, idx + 1, state_dt, hy);
    }
}

// number of time chunks: split only while it at least doubles the number of busy SMs and each
// chunk keeps >= 256 timesteps
int hgrn_num_chunks(int64_t B, int64_t T, int64_t D) {
    const int64_t ctas = B * ((D + HG_BD - 1) / HG_BD);
    int nt = 1;
    while (ctas * nt < 148 && T / (nt * 2) >= 256 && nt < 64) nt *= 2;
    return nt;
}

template <typename TX, typename TG>
size_t hgrn_smem_bytes() {
    return (size_t)HgStages<TX, TG>::value * HG_TS * HG_BD * (sizeof(TX) + sizeof(TG)) + (size_t)2 * HG_TS * HG_BD * sizeof(TX) + 128;
}

// [B][T][D] view with row pitch `ld` elements (batch pitch T*ld), box = one [64 timesteps x 64 channels] tile
int hgrn_make_map(CUtensorMap* map, const void* base, int es, int64_t ld, int64_t B, int64_t T, int64_t D, const char* who) {
    MmfEncodeTiledFn encode = mmf_encode_tiled();
    MMF_REQUIRE(encode != nullptr, MMF_ERR_CUDA, "%s: cuTensorMapEncodeTiled is not available from the driver", who);
    const cuuint64_t gdim[3] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)B};
    const cuuint64_t gstride[2] = {(cuuint64_t)(ld * es), (cuuint64_t)(T * ld * es)};
    const cuuint32_t box[3] = {(cuuint32_t)HG_BD, (cuuint32_t)HG_TS, 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUresult cr = encode(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 3,
                               const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    MMF_REQUIRE(cr == CUDA_SUCCESS, MMF_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed (%d)", who, (int)cr);
    return MMF_OK;
}

template <typename TX, typename TG, int MODE>
int hgrn_launch(const void* x, int64_t ld_x, const void* g, int64_t ld_g, const void* lb, const uint8_t* mask, const void* h0,
                void* ht, int state_dt, void* o, int64_t B, int64_t T, int64_t D, int NT, HgrnWs ws, cudaStream_t st) {
    if (T == 1) {   // a single step: no tiles, no scan
        const int64_t pairs = B * D / 2;
        MMF_CUDA(mmf_launch_pdl(hgrn_step_kernel<TX, TG, MODE>, dim3((unsigned)((pairs + 255) / 256)), dim3(256), 0, st, (const TX*)x,
                                ld_x, (const TG*)g, ld_g, (const TX*)lb, mask, h0, ht, state_dt, (TX*)o, B, (int)D));
        MMF_LAUNCH_CHECK("hgrn_step_kernel");
        return MMF_OK;
    }
    const size_t smem = hgrn_smem_bytes<TX, TG>();
    // chunks start on stage boundaries so that every chunk but the last consists of whole stages
    const int chunk_len = (int)(((T + NT - 1) / NT + HG_TS - 1) / HG_TS * HG_TS);
    CUtensorMap x_map, g_map, o_map;
    int rc = hgrn_make_map(&x_map, x, (int)sizeof(TX), ld_x, B, T, D, "mmf_hgrn");
    if (rc == MMF_OK) rc = hgrn_make_map(&g_map, g, (int)sizeof(TG), ld_g, B, T, D, "mmf_hgrn");
    if (rc == MMF_OK) rc = hgrn_make_map(&o_map, o, (int)sizeof(TX), D, B, T, D, "mmf_hgrn");
    if (rc != MMF_OK) return rc;
    const dim3 grid((unsigned)((D + HG_BD - 1) / HG_BD), (unsigned)NT, (unsigned)B);
    if (NT > 1) {
        auto k1 = hgrn_scan_kernel<TX, TG, MODE, true>;
        MMF_CUDA(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const dim3 grid1(grid.x, (unsigned)(NT - 1), grid.z);
        MMF_CUDA(mmf_launch_pdl(k1, grid1, dim3(HG_THREADS), smem, st, x_map, g_map, o_map, (const TX*)lb, mask, h0,
                                (void*)nullptr, state_dt, (int)T, (int)D, NT, chunk_len, ws));
        MMF_LAUNCH_CHECK("hgrn_scan_kernel<aggregate>");
    }
    auto k2 = hgrn_scan_kernel<TX, TG, MODE, false>;
    MMF_CUDA(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MMF_CUDA(mmf_launch_pdl(k2, grid, dim3(HG_THREADS), smem, st, x_map, g_map, o_map, (const TX*)lb, mask, h0, ht, state_dt,
                            (int)T, (int)D, NT, chunk_len, ws));
    MMF_LAUNCH_CHECK("hgrn_scan_kernel<scan>");
    return MMF_OK;
}

int hgrn_setup_ws(int64_t B, int64_t T, int64_t D, void* workspace, int64_t workspace_bytes, int& NT, HgrnWs& ws,
                  const char* who) {
    NT = hgrn_num_chunks(B, T, D);
    ws = HgrnWs{nullptr, nullptr, nullptr};
    if (NT > 1) {
        const int64_t need = mmf_hgrn_workspace_bytes(B, T, D);
        MMF_REQUIRE(workspace && workspace_bytes >= need, MMF_ERR_WORKSPACE, "%s: workspace of %lld bytes needed, %lld given",
                    who, (long long)need, (long long)workspace_bytes);
        MMF_REQUIRE(mmf_aligned(workspace, 16), MMF_ERR_ALIGN, "%s: workspace must be 16-byte aligned", who);
        ws.h0c = (float*)workspace;
        ws.agg_a = ws.h0c + B * D;
        ws.agg_h = ws.agg_a + B * NT * D;
    }
    return MMF_OK;
}

}  // namespace

extern "C" int64_t mmf_hgrn_workspace_bytes(int64_t B, int64_t T, int64_t D) {
    if (B <= 0 || T <= 0 || D <= 0) return 0;
    const int nt = hgrn_num_chunks(B, T, D);
    if (nt == 1) return 0;
    return (B * D + 2 * B * nt * D) * (int64_t)sizeof(float);
}

extern "C" int mmf_hgrn_scan(const void* x, int x_dtype, const void* g, int g_dtype, const void* h0, void* ht,
                             int state_dtype, void* o, int64_t B, int64_t T, int64_t D, int gate_is_log,
                             void* workspace, int64_t workspace_bytes, void* stream) {
    MMF_REQUIRE(x && g && o, MMF_ERR_BAD_ARG, "mmf_hgrn_scan: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(x_dtype) && mmf_dtype_ok(g_dtype) && mmf_dtype_ok(state_dtype), MMF_ERR_BAD_ARG,
                "mmf_hgrn_scan: unknown dtype");
    MMF_REQUIRE(B >= 0 && T >= 0 && D > 0 && D % 8 == 0, MMF_ERR_BAD_SHAPE, "mmf_hgrn_scan: D must be a multiple of 8");
    MMF_REQUIRE(B < 65536 && T < (1ll << 31) && D < (1ll << 31), MMF_ERR_BAD_SHAPE, "mmf_hgrn_scan: size too large");
    MMF_REQUIRE(mmf_aligned(x, 16) && mmf_aligned(g, 16) && mmf_aligned(o, 16), MMF_ERR_ALIGN,
                "mmf_hgrn_scan: x, g, o must be 16-byte aligned");
    if (B == 0 || T == 0) return MMF_OK;
    int NT;
    HgrnWs ws;
    const int rc0 = hgrn_setup_ws(B, T, D, workspace, workspace_bytes, NT, ws, "mmf_hgrn_scan");
    if (rc0 != MMF_OK) return rc0;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = MMF_OK;
#define HG_GO(TX, TG)                                                                                                  \
    rc = gate_is_log ? hgrn_launch<TX, TG, HG_LOG>(x, D, g, D, nullptr, nullptr, h0, ht, state_dtype, o, B, T, D, NT, ws, st)     \
                     : hgrn_launch<TX, TG, HG_LINEAR>(x, D, g, D, nullptr, nullptr, h0, ht, state_dtype, o, B, T, D, NT, ws, st)
    if (x_dtype == MMF_F32 && g_dtype == MMF_F32) { HG_GO(float, float); }
    else if (x_dtype == MMF_BF16 && g_dtype == MMF_BF16) { HG_GO(__nv_bfloat16, __nv_bfloat16); }
    else if (x_dtype == MMF_BF16 && g_dtype == MMF_F32) { HG_GO(__nv_bfloat16, float); }
    else if (x_dtype == MMF_F16 && g_dtype == MMF_F16) { HG_GO(__half, __half); }
    else if (x_dtype == MMF_F16 && g_dtype == MMF_F32) { HG_GO(__half, float); }
    else return mmf_set_error(MMF_ERR_BAD_ARG, "mmf_hgrn_scan: unsupported dtype pair x=%d g=%d", x_dtype, g_dtype);
#undef HG_GO
    return rc;
}

extern "C" int mmf_hgrn_gated_masked(const void* i_raw, const void* f_raw, int64_t ld, int dtype, const void* lower_bound,
                                     const uint8_t* mask, float* state, void* o, int64_t B, int64_t T, int64_t D,
                                     void* workspace, int64_t workspace_bytes, void* stream) {
    MMF_REQUIRE(i_raw && f_raw && state && o, MMF_ERR_BAD_ARG, "mmf_hgrn_gated: null pointer");
    MMF_REQUIRE(mmf_dtype_ok(dtype), MMF_ERR_BAD_ARG, "mmf_hgrn_gated: unknown dtype %d", dtype);
    MMF_REQUIRE(B >= 0 && B < 65536 && T >= 0 && T < (1ll << 31) && D > 0 && D < (1ll << 31) && D % 8 == 0 && ld >= D,
                MMF_ERR_BAD_SHAPE, "mmf_hgrn_gated: bad sizes (D must be a multiple of 8)");
    const int es = mmf_dtype_size(dtype);
    MMF_REQUIRE(mmf_aligned(i_raw, 16) && mmf_aligned(f_raw, 16) && mmf_aligned(o, 16) && (ld * es) % 16 == 0, MMF_ERR_ALIGN,
                "mmf_hgrn_gated: rows must be 16-byte aligned");
    if (B == 0 || T == 0) return MMF_OK;
    int NT;
    HgrnWs ws;
    const int rc0 = hgrn_setup_ws(B, T, D, workspace, workspace_bytes, NT, ws, "mmf_hgrn_gated");
    if (rc0 != MMF_OK) return rc0;
    int rc = MMF_OK;
    MMF_DISPATCH(dtype, Ty, {
        rc = hgrn_launch<Ty, Ty, HG_RAW>(i_raw, ld, f_raw, ld, lower_bound, mask, state, state, MMF_F32, o, B, T, D, NT, ws,
                                         (cudaStream_t)stream);
    });
    return rc;
}

extern "C" int mmf_hgrn_gated(const void* i_raw, const void* f_raw, int64_t ld, int dtype, const void* lower_bound,
                              float* state, void* o, int64_t B, int64_t T, int64_t D, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    return mmf_hgrn_gated_masked(i_raw, f_raw, ld, dtype, lower_bound, nullptr, state, o, B, T, D, workspace, workspace_bytes, stream);
}

extern "C" int mmf_hgrn_status(int* failed_host) {
    MMF_REQUIRE(failed_host, MMF_ERR_BAD_ARG, "mmf_hgrn_status: null pointer");
    MMF_CUDA(cudaMemcpyFromSymbol(failed_host, g_hgrn_wait_failed, sizeof(int)));
    return MMF_OK;
}
